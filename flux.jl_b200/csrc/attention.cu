// Scaled dot-product attention, flash style: forward with online softmax (no [Lk, Lq, h, B] score tensor in
// HBM), backward by recomputation from the saved log-sum-exp, and on-demand materialisation of the scores.
//
// Layout: Julia q[E, Lq, B] is read as [B][Lq][E]; head h owns features h*d .. (h+1)*d-1 of every row.
// lse is [B][h][Lq].  One block handles one (batch, head, 64-row tile); S / P tiles are 64 x 64.
// Arithmetic is fp32 throughout (FMA pipes), which is what the 1e-4 parity tolerance needs.
#include "common.cuh"

namespace {

constexpr int AT = 256;   // threads: 16 x 16, each owns a 4 x 4 register tile (rows ty+16*i, cols tx+16*j)
constexpr int TS = 64;    // tile size along q and kv
constexpr int PLD = 68;   // row stride of the 64 x 64 P / dS tiles

struct AttnDims {
  int64_t E, Ev, Lq, Lk;
  int H, d, dv, causal;
  float scale;
  // optional extras (the general kernels only): additive bias[j + Lk * i + bias_sh * h + bias_sb * b], dropout on the
  // attention weights (keep-mask element ((b * H + h) * Lq + i) * Lk + j of the Philox stream), cotangent of alpha
  const float* bias;
  int64_t bias_sh, bias_sb;
  const float* dalpha;
  float p_drop, drop_scale;
  uint64_t seed, offset;
};

// the logit of (query i, key j): scaled score plus the additive bias
__device__ __forceinline__ float attn_logit(const AttnDims& D, float s, int64_t b, int h, int64_t i, int64_t j) {
  s *= D.scale;
  if (D.bias != nullptr) s += __ldg(D.bias + b * D.bias_sb + (int64_t)h * D.bias_sh + i * D.Lk + j);
  return s;
}
// what dropout multiplies the attention weight (i, j) with: 0 or 1 / (1 - p)
__device__ __forceinline__ float attn_dropmul(const AttnDims& D, int64_t b, int h, int64_t i, int64_t j) {
  if (D.p_drop <= 0.0f) return 1.0f;
  const uint64_t idx = (uint64_t)(((b * D.H + h) * D.Lq + i) * D.Lk + j);
  return fb_dropout_keep(idx, D.p_drop, D.seed, D.offset) ? D.drop_scale : 0.0f;
}

// dst[r][c] = src[(row0 + r) * ld_src + c] for r < 64, c < LD - 4 (zero padded outside rows < nrows, c < width)
template <int LD>
__device__ __forceinline__ void load_tile(float* __restrict__ dst, const float* __restrict__ src, int64_t ld_src,
                                          int64_t row0, int64_t nrows, int width) {
  constexpr int W = LD - 4;
  for (int e = threadIdx.x; e < TS * W; e += AT) {
    const int r = e / W, c = e % W;
    const int64_t gr = row0 + r;
    dst[r * LD + c] = (gr < nrows && c < width) ? __ldg(src + gr * ld_src + c) : 0.0f;
  }
}

// S[i][j] = sum_c A[ty+16i][c] * B[tx+16j][c], c < kdim (kdim a multiple of 4, zero padded)
template <int LD>
__device__ __forceinline__ void tile_abt(float (&S)[4][4], const float* __restrict__ A, const float* __restrict__ B,
                                         int kdim, int ty, int tx) {
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) S[i][j] = 0.0f;
  for (int c = 0; c < kdim; c += 4) {
    float4 a[4], b[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) a[i] = *(const float4*)(A + (ty + 16 * i) * LD + c);
#pragma unroll
    for (int j = 0; j < 4; ++j) b[j] = *(const float4*)(B + (tx + 16 * j) * LD + c);
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        S[i][j] = fmaf(a[i].x, b[j].x, S[i][j]);
        S[i][j] = fmaf(a[i].y, b[j].y, S[i][j]);
        S[i][j] = fmaf(a[i].z, b[j].z, S[i][j]);
        S[i][j] = fmaf(a[i].w, b[j].w, S[i][j]);
      }
  }
}

// acc[cc][i][.] += sum_j P[ty+16i][j] * V[j][cc*64 + 4*tx + .]      (P is [64][PLD], V is [64][LD])
template <int NC, int LD>
__device__ __forceinline__ void tile_pv(float (&acc)[NC][4][4], const float* __restrict__ P, const float* __restrict__ V,
                                        int ty, int tx) {
  for (int j = 0; j < TS; ++j) {
    float p[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) p[i] = P[(ty + 16 * i) * PLD + j];
#pragma unroll
    for (int cc = 0; cc < NC; ++cc) {
      const float4 v = *(const float4*)(V + j * LD + cc * 64 + 4 * tx);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        acc[cc][i][0] = fmaf(p[i], v.x, acc[cc][i][0]);
        acc[cc][i][1] = fmaf(p[i], v.y, acc[cc][i][1]);
        acc[cc][i][2] = fmaf(p[i], v.z, acc[cc][i][2]);
        acc[cc][i][3] = fmaf(p[i], v.w, acc[cc][i][3]);
      }
    }
  }
}

// acc[cc][jj][.] += sum_i P[i][ty+16jj] * X[i][cc*64 + 4*tx + .]     (P^T * X)
template <int NC, int LD>
__device__ __forceinline__ void tile_ptx(float (&acc)[NC][4][4], const float* __restrict__ P, const float* __restrict__ X,
                                         int ty, int tx) {
  for (int i = 0; i < TS; ++i) {
    float p[4];
#pragma unroll
    for (int jj = 0; jj < 4; ++jj) p[jj] = P[i * PLD + ty + 16 * jj];
#pragma unroll
    for (int cc = 0; cc < NC; ++cc) {
      const float4 x = *(const float4*)(X + i * LD + cc * 64 + 4 * tx);
#pragma unroll
      for (int jj = 0; jj < 4; ++jj) {
        acc[cc][jj][0] = fmaf(p[jj], x.x, acc[cc][jj][0]);
        acc[cc][jj][1] = fmaf(p[jj], x.y, acc[cc][jj][1]);
        acc[cc][jj][2] = fmaf(p[jj], x.z, acc[cc][jj][2]);
        acc[cc][jj][3] = fmaf(p[jj], x.w, acc[cc][jj][3]);
      }
    }
  }
}

__device__ __forceinline__ bool attn_keep(const AttnDims& D, const uint8_t* mask, int64_t i, int64_t j) {
  if (i >= D.Lq || j >= D.Lk) return false;
  if (D.causal && j > i) return false;
  if (mask != nullptr && mask[i * D.Lk + j] == 0) return false;
  return true;
}

// max / sum over the 16 lanes (same ty) that share a row
__device__ __forceinline__ float row16_max(float v) {
#pragma unroll
  for (int o = 8; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float row16_sum(float v) {
#pragma unroll
  for (int o = 8; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// ------------------------------------------------------------------------------------ forward ---
template <int NC>
__global__ void __launch_bounds__(AT)
attn_fwd_kernel(const float* __restrict__ q, const float* __restrict__ k, const float* __restrict__ v,
                const uint8_t* __restrict__ mask, float* __restrict__ o, float* __restrict__ lse, AttnDims D) {
  constexpr int LD = NC * 64 + 4;
  extern __shared__ float sm[];
  float* Qs = sm;
  float* Ks = Qs + TS * LD;
  float* Vs = Ks + TS * LD;
  float* Ps = Vs + TS * LD;
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  const int64_t i0 = (int64_t)blockIdx.x * TS;
  const int h = blockIdx.y;
  const int64_t b = blockIdx.z;
  const float* qb = q + b * D.Lq * D.E + (int64_t)h * D.d;
  const float* kb = k + b * D.Lk * D.E + (int64_t)h * D.d;
  const float* vb = v + b * D.Lk * D.Ev + (int64_t)h * D.dv;
  const int kdim = (D.d + 3) & ~3;

  load_tile<LD>(Qs, qb, D.E, i0, D.Lq, D.d);
  float acc[NC][4][4];
  float m[4], l[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    m[i] = -INFINITY;
    l[i] = 0.0f;
#pragma unroll
    for (int cc = 0; cc < NC; ++cc)
#pragma unroll
      for (int e = 0; e < 4; ++e) acc[cc][i][e] = 0.0f;
  }
  int64_t kv_end = D.Lk;
  if (D.causal && i0 + TS < kv_end) kv_end = i0 + TS;
  for (int64_t j0 = 0; j0 < kv_end; j0 += TS) {
    __syncthreads();
    load_tile<LD>(Ks, kb, D.E, j0, D.Lk, D.d);
    load_tile<LD>(Vs, vb, D.Ev, j0, D.Lk, D.dv);
    __syncthreads();
    float S[4][4];
    tile_abt<LD>(S, Qs, Ks, kdim, ty, tx);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int64_t gi = i0 + ty + 16 * i;
      bool keep[4];
      float mx = -INFINITY;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        keep[j] = attn_keep(D, mask, gi, j0 + tx + 16 * j);
        S[i][j] = keep[j] ? attn_logit(D, S[i][j], b, h, gi, j0 + tx + 16 * j) : -INFINITY;
        mx = fmaxf(mx, S[i][j]);
      }
      mx = row16_max(mx);
      const float m_new = fmaxf(m[i], mx);
      const float m_use = (m_new == -INFINITY) ? 0.0f : m_new;
      const float corr = expf(m[i] - m_use);   // m[i] = -inf gives 0
      float rs = 0.0f;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float p = keep[j] ? expf(S[i][j] - m_use) : 0.0f;
        rs += p;
        // dropout acts on the normalised weights: the row sum keeps every term, the product with V the kept ones
        Ps[(ty + 16 * i) * PLD + tx + 16 * j] = (keep[j] && D.p_drop > 0.0f) ? p * attn_dropmul(D, b, h, gi, j0 + tx + 16 * j) : p;
      }
      rs = row16_sum(rs);
      l[i] = l[i] * corr + rs;
      m[i] = m_new;
#pragma unroll
      for (int cc = 0; cc < NC; ++cc)
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[cc][i][e] *= corr;
    }
    __syncthreads();
    tile_pv<NC, LD>(acc, Ps, Vs, ty, tx);
  }
  float* ob = o + b * D.Lq * D.Ev + (int64_t)h * D.dv;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int64_t gi = i0 + ty + 16 * i;
    if (gi >= D.Lq) continue;
    const float inv = l[i] > 0.0f ? 1.0f / l[i] : 0.0f;
#pragma unroll
    for (int cc = 0; cc < NC; ++cc)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int c = cc * 64 + 4 * tx + e;
        if (c < D.dv) ob[gi * D.Ev + c] = acc[cc][i][e] * inv;
      }
    if (tx == 0) lse[(b * D.H + h) * D.Lq + gi] = (l[i] > 0.0f) ? m[i] + logf(l[i]) : -INFINITY;
  }
}

// dlt[b][h][i] = sum_c dO[b][i][h*dv + c] * O[b][i][h*dv + c]; one warp per (b, i, h)
__global__ void __launch_bounds__(AT)
attn_delta_kernel(const float* __restrict__ o, const float* __restrict__ dout, float* __restrict__ dlt, AttnDims D,
                  int64_t B) {
  const int lane = threadIdx.x & 31;
  const int64_t w = (int64_t)blockIdx.x * (AT / 32) + (threadIdx.x >> 5);
  const int64_t total = B * D.Lq * D.H;
  if (w >= total) return;
  const int h = (int)(w % D.H);
  const int64_t bi = w / D.H;            // b * Lq + i
  const int64_t b = bi / D.Lq, i = bi % D.Lq;
  const float* op = o + bi * D.Ev + (int64_t)h * D.dv;
  const float* dp = dout + bi * D.Ev + (int64_t)h * D.dv;
  float s = 0.0f;
  for (int c = lane; c < D.dv; c += 32) s = fmaf(op[c], dp[c], s);
  s = fb_warp_sum(s);
  if (lane == 0) dlt[(b * D.H + h) * D.Lq + i] = s;
}

// P and dS tiles for (q tile i0, kv tile j0) from staged Q, K, V, dO.
template <int LD>
__device__ __forceinline__ void recompute_p_ds(const AttnDims& D, const uint8_t* mask, const float* Qs, const float* Ks,
                                               const float* Vs, const float* dOs, const float* lse_bh,
                                               const float* dlt_bh, int64_t i0, int64_t j0, int ty, int tx,
                                               float* Ps, float* dSs, int64_t b, int h) {
  const int kdim = (D.d + 3) & ~3, vdim = (D.dv + 3) & ~3;
  float S[4][4], dP[4][4];
  tile_abt<LD>(S, Qs, Ks, kdim, ty, tx);
  tile_abt<LD>(dP, dOs, Vs, vdim, ty, tx);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int64_t gi = i0 + ty + 16 * i;
    const float ls = gi < D.Lq ? lse_bh[gi] : -INFINITY;
    const float dl = gi < D.Lq ? dlt_bh[gi] : 0.0f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const bool keep = attn_keep(D, mask, gi, j0 + tx + 16 * j) && (ls != -INFINITY);
      const int64_t gj = j0 + tx + 16 * j;
      const float p = keep ? expf(attn_logit(D, S[i][j], b, h, gi, gj) - ls) : 0.0f;
      const float dm = keep ? attn_dropmul(D, b, h, gi, gj) : 0.0f;
      float dp = dP[i][j];
      if (D.dalpha != nullptr && keep) dp += __ldg(D.dalpha + ((b * D.H + h) * D.Lq + gi) * D.Lk + gj);
      if (Ps) Ps[(ty + 16 * i) * PLD + tx + 16 * j] = p * dm;          // the weights that multiplied V
      dSs[(ty + 16 * i) * PLD + tx + 16 * j] = p * (dp * dm - dl);
    }
  }
}

// ------------------------------------------------------------------------- backward: dK, dV ---
template <int NC>
__global__ void __launch_bounds__(AT)
attn_bwd_dkdv_kernel(const float* __restrict__ q, const float* __restrict__ k, const float* __restrict__ v,
                     const uint8_t* __restrict__ mask, const float* __restrict__ lse, const float* __restrict__ dlt,
                     const float* __restrict__ dout, float* __restrict__ dk, float* __restrict__ dv, AttnDims D) {
  constexpr int LD = NC * 64 + 4;
  extern __shared__ float sm[];
  float* Ks = sm;
  float* Vs = Ks + TS * LD;
  float* Qs = Vs + TS * LD;
  float* dOs = Qs + TS * LD;
  float* Ps = dOs + TS * LD;
  float* dSs = Ps + TS * PLD;
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  const int64_t j0 = (int64_t)blockIdx.x * TS;
  const int h = blockIdx.y;
  const int64_t b = blockIdx.z;
  const float* qb = q + b * D.Lq * D.E + (int64_t)h * D.d;
  const float* kb = k + b * D.Lk * D.E + (int64_t)h * D.d;
  const float* vb = v + b * D.Lk * D.Ev + (int64_t)h * D.dv;
  const float* dob = dout + b * D.Lq * D.Ev + (int64_t)h * D.dv;
  const float* lse_bh = lse + (b * D.H + h) * D.Lq;
  const float* dlt_bh = dlt + (b * D.H + h) * D.Lq;
  load_tile<LD>(Ks, kb, D.E, j0, D.Lk, D.d);
  load_tile<LD>(Vs, vb, D.Ev, j0, D.Lk, D.dv);
  float adk[NC][4][4], adv[NC][4][4];
#pragma unroll
  for (int cc = 0; cc < NC; ++cc)
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int e = 0; e < 4; ++e) { adk[cc][i][e] = 0.0f; adv[cc][i][e] = 0.0f; }
  const int64_t i_begin = D.causal ? j0 : 0;   // queries i < j0 never see keys of this tile
  for (int64_t i0 = i_begin; i0 < D.Lq; i0 += TS) {
    __syncthreads();
    load_tile<LD>(Qs, qb, D.E, i0, D.Lq, D.d);
    load_tile<LD>(dOs, dob, D.Ev, i0, D.Lq, D.dv);
    __syncthreads();
    recompute_p_ds<LD>(D, mask, Qs, Ks, Vs, dOs, lse_bh, dlt_bh, i0, j0, ty, tx, Ps, dSs, b, h);
    __syncthreads();
    tile_ptx<NC, LD>(adv, Ps, dOs, ty, tx);
    tile_ptx<NC, LD>(adk, dSs, Qs, ty, tx);
  }
  float* dkb = dk + b * D.Lk * D.E + (int64_t)h * D.d;
  float* dvb = dv + b * D.Lk * D.Ev + (int64_t)h * D.dv;
#pragma unroll
  for (int jj = 0; jj < 4; ++jj) {
    const int64_t gj = j0 + ty + 16 * jj;
    if (gj >= D.Lk) continue;
#pragma unroll
    for (int cc = 0; cc < NC; ++cc)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int c = cc * 64 + 4 * tx + e;
        if (c < D.d) dkb[gj * D.E + c] = adk[cc][jj][e] * D.scale;
        if (c < D.dv) dvb[gj * D.Ev + c] = adv[cc][jj][e];
      }
  }
}

// ----------------------------------------------------------------------------- backward: dQ ---
template <int NC>
__global__ void __launch_bounds__(AT)
attn_bwd_dq_kernel(const float* __restrict__ q, const float* __restrict__ k, const float* __restrict__ v,
                   const uint8_t* __restrict__ mask, const float* __restrict__ lse, const float* __restrict__ dlt,
                   const float* __restrict__ dout, float* __restrict__ dq, AttnDims D) {
  constexpr int LD = NC * 64 + 4;
  extern __shared__ float sm[];
  float* Qs = sm;
  float* dOs = Qs + TS * LD;
  float* Ks = dOs + TS * LD;
  float* Vs = Ks + TS * LD;
  float* dSs = Vs + TS * LD;
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  const int64_t i0 = (int64_t)blockIdx.x * TS;
  const int h = blockIdx.y;
  const int64_t b = blockIdx.z;
  const float* qb = q + b * D.Lq * D.E + (int64_t)h * D.d;
  const float* kb = k + b * D.Lk * D.E + (int64_t)h * D.d;
  const float* vb = v + b * D.Lk * D.Ev + (int64_t)h * D.dv;
  const float* dob = dout + b * D.Lq * D.Ev + (int64_t)h * D.dv;
  const float* lse_bh = lse + (b * D.H + h) * D.Lq;
  const float* dlt_bh = dlt + (b * D.H + h) * D.Lq;
  load_tile<LD>(Qs, qb, D.E, i0, D.Lq, D.d);
  load_tile<LD>(dOs, dob, D.Ev, i0, D.Lq, D.dv);
  float adq[NC][4][4];
#pragma unroll
  for (int cc = 0; cc < NC; ++cc)
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int e = 0; e < 4; ++e) adq[cc][i][e] = 0.0f;
  int64_t kv_end = D.Lk;
  if (D.causal && i0 + TS < kv_end) kv_end = i0 + TS;
  for (int64_t j0 = 0; j0 < kv_end; j0 += TS) {
    __syncthreads();
    load_tile<LD>(Ks, kb, D.E, j0, D.Lk, D.d);
    load_tile<LD>(Vs, vb, D.Ev, j0, D.Lk, D.dv);
    __syncthreads();
    recompute_p_ds<LD>(D, mask, Qs, Ks, Vs, dOs, lse_bh, dlt_bh, i0, j0, ty, tx, nullptr, dSs, b, h);
    __syncthreads();
    tile_pv<NC, LD>(adq, dSs, Ks, ty, tx);
  }
  float* dqb = dq + b * D.Lq * D.E + (int64_t)h * D.d;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int64_t gi = i0 + ty + 16 * i;
    if (gi >= D.Lq) continue;
#pragma unroll
    for (int cc = 0; cc < NC; ++cc)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int c = cc * 64 + 4 * tx + e;
        if (c < D.d) dqb[gi * D.E + c] = adq[cc][i][e] * D.scale;
      }
  }
}

// --------------------------------------------------------------------- scores on demand ---
// alpha memory is [B][h][Lq][Lk] (Julia alpha[Lk, Lq, h, B]); grid (kv tiles, q tiles, B*h)
template <int NC>
__global__ void __launch_bounds__(AT)
attn_scores_kernel(const float* __restrict__ q, const float* __restrict__ k, const uint8_t* __restrict__ mask,
                   const float* __restrict__ lse, float* __restrict__ alpha, float* __restrict__ extra_dlt, AttnDims D) {
  // With extra_dlt the kernel does not write alpha: it adds sum_j alpha_ij * dalpha_ij to extra_dlt[b][h][i] (the
  // share of an alpha cotangent in the softmax backward's row term).
  constexpr int LD = NC * 64 + 4;
  extern __shared__ float sm[];
  float* Qs = sm;
  float* Ks = Qs + TS * LD;
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  float row_extra[4] = {0.0f, 0.0f, 0.0f, 0.0f};
  const int64_t j0 = (int64_t)blockIdx.x * TS, i0 = (int64_t)blockIdx.y * TS;
  const int64_t bh = blockIdx.z;
  const int64_t b = bh / D.H;
  const int h = (int)(bh % D.H);
  load_tile<LD>(Qs, q + b * D.Lq * D.E + (int64_t)h * D.d, D.E, i0, D.Lq, D.d);
  load_tile<LD>(Ks, k + b * D.Lk * D.E + (int64_t)h * D.d, D.E, j0, D.Lk, D.d);
  __syncthreads();
  float S[4][4];
  tile_abt<LD>(S, Qs, Ks, (D.d + 3) & ~3, ty, tx);
  const float* lse_bh = lse + bh * D.Lq;
  float* ab = alpha + bh * D.Lq * D.Lk;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int64_t gi = i0 + ty + 16 * i;
    if (gi >= D.Lq) continue;
    const float ls = lse_bh[gi];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int64_t gj = j0 + tx + 16 * j;
      if (gj >= D.Lk) continue;
      const bool keep = attn_keep(D, mask, gi, gj) && (ls != -INFINITY);
      const float a = keep ? expf(attn_logit(D, S[i][j], b, h, gi, gj) - ls) * attn_dropmul(D, b, h, gi, gj) : 0.0f;
      if (extra_dlt != nullptr) {
        // contribution of the alpha cotangent to delta_i = sum_j alpha_ij * dalpha_ij (alpha after dropout)
        row_extra[i] += a * __ldg(D.dalpha + (bh * D.Lq + gi) * D.Lk + gj);
      } else {
        ab[gi * D.Lk + gj] = a;
      }
    }
  }
  if (extra_dlt != nullptr) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float r = row16_sum(row_extra[i]);
      const int64_t gi = i0 + ty + 16 * i;
      if (tx == 0 && gi < D.Lq && r != 0.0f) atomicAdd(extra_dlt + bh * D.Lq + gi, r);
    }
  }
}

int32_t attn_make_dims(const char* fn, AttnDims* D, int64_t e_dim, int64_t ev_dim, int64_t lq, int64_t lk,
                       int64_t batch, int32_t nheads, int32_t causal) {
  FB_REQUIRE(nheads >= 1 && e_dim >= 1 && ev_dim >= 1 && lq >= 0 && lk >= 0 && batch >= 0, FB_ERR_SHAPE,
             "%s: bad shape E=%lld Ev=%lld Lq=%lld Lk=%lld B=%lld heads=%d", fn, (long long)e_dim, (long long)ev_dim,
             (long long)lq, (long long)lk, (long long)batch, nheads);
  FB_REQUIRE(e_dim % nheads == 0, FB_ERR_SHAPE, "%s: qk_dim = %lld should be divisible by nheads = %d", fn,
             (long long)e_dim, nheads);
  FB_REQUIRE(ev_dim % nheads == 0, FB_ERR_SHAPE, "%s: v_dim = %lld should be divisible by nheads = %d", fn,
             (long long)ev_dim, nheads);
  FB_REQUIRE(e_dim / nheads <= 128 && ev_dim / nheads <= 128, FB_ERR_UNSUPPORTED,
             "%s: head dimension above 128 is not supported", fn);
  FB_REQUIRE(nheads <= 65535 && batch <= 65535 && batch * nheads <= 65535, FB_ERR_SHAPE, "%s: batch * heads too large", fn);
  D->E = e_dim; D->Ev = ev_dim; D->Lq = lq; D->Lk = lk; D->H = nheads;
  D->d = (int)(e_dim / nheads); D->dv = (int)(ev_dim / nheads); D->causal = causal ? 1 : 0;
  D->scale = 1.0f / sqrtf((float)D->d);
  D->bias = nullptr; D->bias_sh = 0; D->bias_sb = 0; D->dalpha = nullptr;
  D->p_drop = 0.0f; D->drop_scale = 1.0f; D->seed = 0; D->offset = 0;
  return FB_OK;
}

// additive bias and dropout of the extended entry points
int32_t attn_set_extras(const char* fn, AttnDims* D, const float* bias, int64_t bias_sh, int64_t bias_sb, float p_drop, uint64_t seed,
                        uint64_t offset) {
  FB_REQUIRE(p_drop >= 0.0f && p_drop < 1.0f, FB_ERR_INVALID_ARG, "%s: dropout probability %g is outside [0, 1)", fn, (double)p_drop);
  FB_REQUIRE(bias_sh >= 0 && bias_sb >= 0, FB_ERR_INVALID_ARG, "%s: negative bias stride", fn);
  D->bias = bias; D->bias_sh = bias ? bias_sh : 0; D->bias_sb = bias ? bias_sb : 0;
  D->p_drop = p_drop; D->drop_scale = 1.0f / (1.0f - p_drop); D->seed = seed; D->offset = offset;
  return FB_OK;
}
bool attn_has_extras(const AttnDims& D) { return D.bias != nullptr || D.p_drop > 0.0f || D.dalpha != nullptr; }

}  // namespace

FB_API int32_t fb_attn_fwd(fb_ctx* ctx, void* stream_, const float* q, const float* k, const float* v,
                           const uint8_t* mask, float* o, float* lse, int64_t e_dim, int64_t ev_dim, int64_t lq,
                           int64_t lk, int64_t batch, int32_t nheads, int32_t causal) {
  return fb_attn_fwd_ex(ctx, stream_, q, k, v, mask, nullptr, 0, 0, 0.0f, 0, 0, o, lse, e_dim, ev_dim, lq, lk, batch, nheads, causal);
}

FB_API int32_t fb_attn_fwd_ex(fb_ctx* ctx, void* stream_, const float* q, const float* k, const float* v, const uint8_t* mask,
                              const float* bias, int64_t bias_stride_h, int64_t bias_stride_b, float p_drop, uint64_t seed,
                              uint64_t offset, float* o, float* lse, int64_t e_dim, int64_t ev_dim, int64_t lq, int64_t lk,
                              int64_t batch, int32_t nheads, int32_t causal) {
  FB_CHECK_CTX(ctx);
  cudaStream_t stream = (cudaStream_t)stream_;
  AttnDims D;
  int32_t st = attn_make_dims("fb_attn_fwd", &D, e_dim, ev_dim, lq, lk, batch, nheads, causal);
  if (st != FB_OK) return st;
  st = attn_set_extras("fb_attn_fwd", &D, bias, bias_stride_h, bias_stride_b, p_drop, seed, offset);
  if (st != FB_OK) return st;
  if (lq == 0 || batch == 0) return FB_OK;
  FB_REQUIRE(q && k && v && o && lse, FB_ERR_INVALID_ARG, "fb_attn_fwd: NULL pointer");
  // head size 64 without an explicit mask, bias or dropout runs on the tensor cores
  st = attn_has_extras(D) ? FB_ERR_UNSUPPORTED
                          : fb_attn_fwd_tc(ctx, stream, q, k, v, mask, o, lse, e_dim, ev_dim, lq, lk, batch, nheads, causal);
  if (st != FB_ERR_UNSUPPORTED) return st;
  const int nc = (D.d > 64 || D.dv > 64) ? 2 : 1;
  const size_t smem = (size_t)(3 * TS * (nc * 64 + 4) + TS * PLD) * sizeof(float);
  dim3 grid((unsigned)((lq + TS - 1) / TS), (unsigned)nheads, (unsigned)batch);
  if (nc == 1) {
    FB_CUDA(cudaFuncSetAttribute(attn_fwd_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    attn_fwd_kernel<1><<<grid, AT, smem, stream>>>(q, k, v, mask, o, lse, D);
  } else {
    FB_CUDA(cudaFuncSetAttribute(attn_fwd_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    attn_fwd_kernel<2><<<grid, AT, smem, stream>>>(q, k, v, mask, o, lse, D);
  }
  FB_LAUNCH_CHECK();
  return FB_OK;
}

FB_API int32_t fb_attn_bwd(fb_ctx* ctx, void* stream_, const float* q, const float* k, const float* v,
                           const uint8_t* mask, const float* o, const float* lse, const float* dout, float* dq,
                           float* dk, float* dv, int64_t e_dim, int64_t ev_dim, int64_t lq, int64_t lk, int64_t batch,
                           int32_t nheads, int32_t causal) {
  return fb_attn_bwd_ex(ctx, stream_, q, k, v, mask, nullptr, 0, 0, 0.0f, 0, 0, o, lse, dout, nullptr, dq, dk, dv, e_dim, ev_dim, lq, lk,
                        batch, nheads, causal);
}

FB_API int32_t fb_attn_bwd_ex(fb_ctx* ctx, void* stream_, const float* q, const float* k, const float* v, const uint8_t* mask,
                              const float* bias, int64_t bias_stride_h, int64_t bias_stride_b, float p_drop, uint64_t seed,
                              uint64_t offset, const float* o, const float* lse, const float* dout, const float* dalpha, float* dq,
                              float* dk, float* dv, int64_t e_dim, int64_t ev_dim, int64_t lq, int64_t lk, int64_t batch,
                              int32_t nheads, int32_t causal) {
  FB_CHECK_CTX(ctx);
  cudaStream_t stream = (cudaStream_t)stream_;
  AttnDims D;
  int32_t st = attn_make_dims("fb_attn_bwd", &D, e_dim, ev_dim, lq, lk, batch, nheads, causal);
  if (st != FB_OK) return st;
  st = attn_set_extras("fb_attn_bwd", &D, bias, bias_stride_h, bias_stride_b, p_drop, seed, offset);
  if (st != FB_OK) return st;
  D.dalpha = dalpha;
  if (batch == 0) return FB_OK;
  FB_REQUIRE(lq >= 1 && lk >= 1, FB_ERR_SHAPE, "fb_attn_bwd: empty sequence");
  FB_REQUIRE(q && k && v && o && lse && dout && dq && dk && dv, FB_ERR_INVALID_ARG, "fb_attn_bwd: NULL pointer");
  float* dlt = (float*)fb_scratch(ctx, stream, (size_t)(batch * nheads * lq) * sizeof(float));
  if (!dlt) return FB_ERR_ALLOC;
  const int64_t warps = batch * lq * nheads;
  attn_delta_kernel<<<(unsigned)((warps + AT / 32 - 1) / (AT / 32)), AT, 0, stream>>>(o, dout, dlt, D, batch);
  FB_LAUNCH_CHECK();
  const int nc = (D.d > 64 || D.dv > 64) ? 2 : 1;
  const int ld = nc * 64 + 4;
  if (dalpha != nullptr) {
    // a cotangent of the attention weights adds sum_j alpha_ij * dalpha_ij to the row term of the softmax backward
    FB_REQUIRE((lq + TS - 1) / TS <= 65535, FB_ERR_SHAPE, "fb_attn_bwd: query length too large");
    const int ncs = D.d > 64 ? 2 : 1;
    const size_t smem_s = (size_t)(2 * TS * (ncs * 64 + 4)) * sizeof(float);
    dim3 grid_s((unsigned)((lk + TS - 1) / TS), (unsigned)((lq + TS - 1) / TS), (unsigned)(batch * nheads));
    if (ncs == 1) {
      FB_CUDA(cudaFuncSetAttribute(attn_scores_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_s));
      attn_scores_kernel<1><<<grid_s, AT, smem_s, stream>>>(q, k, mask, lse, nullptr, dlt, D);
    } else {
      FB_CUDA(cudaFuncSetAttribute(attn_scores_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_s));
      attn_scores_kernel<2><<<grid_s, AT, smem_s, stream>>>(q, k, mask, lse, nullptr, dlt, D);
    }
    FB_LAUNCH_CHECK();
  }
  const bool extras = attn_has_extras(D);
  const size_t smem_kv = (size_t)(4 * TS * ld + 2 * TS * PLD) * sizeof(float);
  const size_t smem_q = (size_t)(4 * TS * ld + TS * PLD) * sizeof(float);
  dim3 grid_kv((unsigned)((lk + TS - 1) / TS), (unsigned)nheads, (unsigned)batch);
  dim3 grid_q((unsigned)((lq + TS - 1) / TS), (unsigned)nheads, (unsigned)batch);
  if (nc == 1) {
    FB_CUDA(cudaFuncSetAttribute(attn_bwd_dkdv_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_kv));
    FB_CUDA(cudaFuncSetAttribute(attn_bwd_dq_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_q));
    // dK / dV on the tensor cores where the shape allows (head size 64, no explicit mask, at most 2048 queries)
    st = extras ? FB_ERR_UNSUPPORTED
                : fb_attn_bwd_dkdv_tc(ctx, stream, q, k, v, mask, lse, dlt, dout, dk, dv, e_dim, ev_dim, lq, lk, batch, nheads, causal);
    if (st == FB_ERR_UNSUPPORTED) {
      attn_bwd_dkdv_kernel<1><<<grid_kv, AT, smem_kv, stream>>>(q, k, v, mask, lse, dlt, dout, dk, dv, D);
      FB_LAUNCH_CHECK();
    } else if (st != FB_OK) {
      return st;
    }
    // dQ on the tensor cores where the shape allows (head size 64, no explicit mask, at most 2048 keys)
    st = extras ? FB_ERR_UNSUPPORTED
                : fb_attn_bwd_dq_tc(ctx, stream, q, k, v, mask, lse, dlt, dout, dq, e_dim, ev_dim, lq, lk, batch, nheads, causal);
    if (st != FB_ERR_UNSUPPORTED) return st;
    attn_bwd_dq_kernel<1><<<grid_q, AT, smem_q, stream>>>(q, k, v, mask, lse, dlt, dout, dq, D);
  } else {
    FB_CUDA(cudaFuncSetAttribute(attn_bwd_dkdv_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_kv));
    FB_CUDA(cudaFuncSetAttribute(attn_bwd_dq_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_q));
    attn_bwd_dkdv_kernel<2><<<grid_kv, AT, smem_kv, stream>>>(q, k, v, mask, lse, dlt, dout, dk, dv, D);
    FB_LAUNCH_CHECK();
    attn_bwd_dq_kernel<2><<<grid_q, AT, smem_q, stream>>>(q, k, v, mask, lse, dlt, dout, dq, D);
  }
  FB_LAUNCH_CHECK();
  return FB_OK;
}

FB_API int32_t fb_attn_scores(fb_ctx* ctx, void* stream_, const float* q, const float* k, const uint8_t* mask,
                              const float* lse, float* alpha, int64_t e_dim, int64_t lq, int64_t lk, int64_t batch,
                              int32_t nheads, int32_t causal) {
  return fb_attn_scores_ex(ctx, stream_, q, k, mask, nullptr, 0, 0, 0.0f, 0, 0, lse, alpha, e_dim, lq, lk, batch, nheads, causal);
}

FB_API int32_t fb_attn_scores_ex(fb_ctx* ctx, void* stream_, const float* q, const float* k, const uint8_t* mask, const float* bias,
                                 int64_t bias_stride_h, int64_t bias_stride_b, float p_drop, uint64_t seed, uint64_t offset,
                                 const float* lse, float* alpha, int64_t e_dim, int64_t lq, int64_t lk, int64_t batch,
                                 int32_t nheads, int32_t causal) {
  FB_CHECK_CTX(ctx);
  cudaStream_t stream = (cudaStream_t)stream_;
  AttnDims D;
  int32_t st = attn_make_dims("fb_attn_scores", &D, e_dim, e_dim, lq, lk, batch, nheads, causal);
  if (st != FB_OK) return st;
  st = attn_set_extras("fb_attn_scores", &D, bias, bias_stride_h, bias_stride_b, p_drop, seed, offset);
  if (st != FB_OK) return st;
  if (lq == 0 || lk == 0 || batch == 0) return FB_OK;
  FB_REQUIRE(q && k && lse && alpha, FB_ERR_INVALID_ARG, "fb_attn_scores: NULL pointer");
  FB_REQUIRE((lq + TS - 1) / TS <= 65535, FB_ERR_SHAPE, "fb_attn_scores: query length too large");
  const int nc = D.d > 64 ? 2 : 1;
  const size_t smem = (size_t)(2 * TS * (nc * 64 + 4)) * sizeof(float);
  dim3 grid((unsigned)((lk + TS - 1) / TS), (unsigned)((lq + TS - 1) / TS), (unsigned)(batch * nheads));
  if (nc == 1) {
    FB_CUDA(cudaFuncSetAttribute(attn_scores_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    attn_scores_kernel<1><<<grid, AT, smem, stream>>>(q, k, mask, lse, alpha, nullptr, D);
  } else {
    FB_CUDA(cudaFuncSetAttribute(attn_scores_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    attn_scores_kernel<2><<<grid, AT, smem, stream>>>(q, k, mask, lse, alpha, nullptr, D);
  }
  FB_LAUNCH_CHECK();
  return FB_OK;
}
