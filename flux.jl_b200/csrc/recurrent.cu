// Recurrence over LSTMCell / GRUCell: fused scan forward and BPTT backward.
//
// Layout: Julia x[in, T, B] is read as [B][T][in]; row (b, t) = b*T + t.  out[H, T, B] likewise.
// Forward:  (1) one GEMM over all T*B columns for the input projection Gx = x*Wi' + b,
//           (2) T step kernels; a block owns HU hidden units (NG*HU rows of Wh, staged in shared memory),
//               streams h_{t-1} through shared memory, and finishes the gate math for its units in place.
// Backward: T step kernels in reverse (gate derivatives, then dh_{t-1} = Wh' * dgates), followed by three
//           GEMMs over all T*B columns for dWi, dWh and dx.
// Steps are ordered by the stream (one launch per step), so no kernel ever waits on another block.
#include <stdlib.h>

#include "common.cuh"

namespace {

constexpr int RT = 256;      // threads per block
constexpr int BC = 64;       // batch columns per pass
constexpr int KC = 128;      // k values staged per pass
constexpr int HS = KC + 4;   // padded row stride of the staged h tile (float4-aligned, conflict-free)

// acc[r] += sum_k Ws[r][k] * v[b][k] for this thread's b and its quarter of every k-chunk.
//   Ws: shared [NR][kp] (kp = K rounded up to KC, zero padded); v: global rows of length K at stride ldv
//   (NULL = all zeros); vs: shared [BC][HS] staging tile.
template <int NR>
__device__ __forceinline__ void rows_times_vec(const float* __restrict__ Ws, int kp, const float* __restrict__ v,
                                               int64_t ldv, int K, int b0, int B, float* __restrict__ vs,
                                               float* acc) {
  const int b = threadIdx.x & (BC - 1), kq = threadIdx.x >> 6;
#pragma unroll
  for (int r = 0; r < NR; ++r) acc[r] = 0.0f;
  if (v == nullptr) return;
  for (int kc = 0; kc < kp; kc += KC) {
    __syncthreads();
    // stage v[b0 .. b0+BC)[kc .. kc+KC): 32 consecutive threads read 128 consecutive floats
    for (int e = threadIdx.x; e < BC * KC; e += RT) {
      const int bb = e / KC, kk = e % KC;
      const int gb = b0 + bb, gk = kc + kk;
      vs[bb * HS + kk] = (gb < B && gk < K) ? __ldg(v + (int64_t)gb * ldv + gk) : 0.0f;
    }
    __syncthreads();
    const float4* vrow = (const float4*)(vs + b * HS + kq * (KC / 4));
#pragma unroll 2
    for (int k4 = 0; k4 < KC / 16; ++k4) {
      const float4 hv = vrow[k4];
      const int kbase = kc + kq * (KC / 4) + k4 * 4;
#pragma unroll
      for (int r = 0; r < NR; ++r) {
        const float4 w = *(const float4*)(Ws + r * kp + kbase);
        acc[r] = fmaf(w.x, hv.x, acc[r]);
        acc[r] = fmaf(w.y, hv.y, acc[r]);
        acc[r] = fmaf(w.z, hv.z, acc[r]);
        acc[r] = fmaf(w.w, hv.w, acc[r]);
      }
    }
  }
}

// Sum the four k-quarter partials through shared memory: red[kq][b][r]; result for (b, r) in red[0][b][r].
template <int NR>
__device__ __forceinline__ void reduce_quarters(float* __restrict__ red, const float* acc) {
  const int b = threadIdx.x & (BC - 1), kq = threadIdx.x >> 6;
  __syncthreads();
#pragma unroll
  for (int r = 0; r < NR; ++r) red[(kq * BC + b) * (NR + 1) + r] = acc[r];
  __syncthreads();
  for (int e = threadIdx.x; e < BC * NR; e += RT) {
    const int bb = e / NR, r = e % NR;
    float s = 0.0f;
#pragma unroll
    for (int q = 0; q < 4; ++q) s += red[(q * BC + bb) * (NR + 1) + r];
    red[bb * (NR + 1) + r] = s;   // (0, bb, r) is only read by this thread in this pass
  }
  __syncthreads();
}

// Stage the NG*HU rows of Wh that belong to units [u0, u0+HU) into shared memory, zero padded to kp.
// Wh memory is [H (k)][NG*H (row)] (Julia Wh[NG*H, H]); row r = g*H + u.
template <int NG, int HU>
__device__ __forceinline__ void stage_w_rows(float* __restrict__ Ws, int kp, const float* __restrict__ Wh, int H, int u0) {
  for (int e = threadIdx.x; e < NG * HU * kp; e += RT) {
    const int k = e / (NG * HU), rr = e % (NG * HU);   // rr fastest: consecutive threads read neighbouring units
    const int g = rr / HU, u = rr % HU;
    float w = 0.0f;
    if (k < H && u0 + u < H) w = __ldg(Wh + (int64_t)k * (NG * H) + g * H + u0 + u);
    Ws[rr * kp + k] = w;
  }
}

// ------------------------------------------------------------------------------- LSTM forward step ---
template <int HU>
__global__ void __launch_bounds__(RT)
lstm_fwd_step_kernel(const float* __restrict__ Wh, const float* __restrict__ gx, const float* __restrict__ hprev,
                     int64_t ldh, const float* __restrict__ cprev, int64_t ldc, float* __restrict__ out_t,
                     int64_t ldo, float* __restrict__ gates_t, float* __restrict__ c_t, int64_t ldcache_g,
                     int64_t ldcache_c, float* __restrict__ hT, float* __restrict__ cT, int H, int B, int64_t ldgx) {
  extern __shared__ float sm[];
  const int kp = (H + KC - 1) / KC * KC;
  constexpr int NR = 4 * HU;
  float* Ws = sm;                         // [NR][kp]
  float* vs = Ws + NR * kp;               // [BC][HS]
  float* red = vs + BC * HS;              // [4][BC][NR+1]
  const int u0 = blockIdx.x * HU;
  stage_w_rows<4, HU>(Ws, kp, Wh, H, u0);
  for (int b0 = 0; b0 < B; b0 += BC) {
    float acc[NR];
    rows_times_vec<NR>(Ws, kp, hprev, ldh, H, b0, B, vs, acc);
    reduce_quarters<NR>(red, acc);
    for (int e = threadIdx.x; e < BC * HU; e += RT) {
      const int bb = e / HU, u = e % HU;
      const int gb = b0 + bb, gu = u0 + u;
      if (gb < B && gu < H) {
        const float* pre = red + bb * (NR + 1);
        const float* gxr = gx + (int64_t)gb * ldgx;
        const float zi = pre[0 * HU + u] + gxr[gu];
        const float zf = pre[1 * HU + u] + gxr[H + gu];
        const float zg = pre[2 * HU + u] + gxr[2 * H + gu];
        const float zo = pre[3 * HU + u] + gxr[3 * H + gu];
        const float ig = 1.0f / (1.0f + expf(-zi)), fg = 1.0f / (1.0f + expf(-zf));
        const float gg = tanhf(zg), og = 1.0f / (1.0f + expf(-zo));
        const float cp = cprev ? cprev[(int64_t)gb * ldc + gu] : 0.0f;
        const float cn = fg * cp + ig * gg;
        const float hn = og * tanhf(cn);
        out_t[(int64_t)gb * ldo + gu] = hn;
        if (gates_t) {
          float* gr = gates_t + (int64_t)gb * ldcache_g;
          gr[gu] = ig; gr[H + gu] = fg; gr[2 * H + gu] = gg; gr[3 * H + gu] = og;
        }
        c_t[(int64_t)gb * ldcache_c + gu] = cn;
        if (hT) { hT[(int64_t)gb * H + gu] = hn; cT[(int64_t)gb * H + gu] = cn; }
      }
    }
  }
}

// gate derivatives for step t, in place over the cached gates:
//   dh = dout_t + dh_rec; do = dh*tanh(c); dc += dh*o*(1-tanh(c)^2); di = dc*g; dg = dc*i; df = dc*c_prev
//   gates <- (di*i*(1-i), df*f*(1-f), dg*(1-g^2), do*o*(1-o)); dc_prev = dc*f
__global__ void __launch_bounds__(RT)
lstm_bwd_gates_kernel(float* __restrict__ gates_t, int64_t ldg, const float* __restrict__ c_t,
                      const float* __restrict__ c_prev, int64_t ldc, int64_t ldcp,
                      const float* __restrict__ dout_t, int64_t ldo, const float* __restrict__ dh_rec, int nparts,
                      float* __restrict__ dc, int H, int B) {
  const int64_t total = (int64_t)B * H;
  for (int64_t e = (int64_t)blockIdx.x * RT + threadIdx.x; e < total; e += (int64_t)gridDim.x * RT) {
    const int b = (int)(e / H), u = (int)(e % H);
    float* gr = gates_t + (int64_t)b * ldg;
    const float ig = gr[u], fg = gr[H + u], gg = gr[2 * H + u], og = gr[3 * H + u];
    const float tc = tanhf(c_t[(int64_t)b * ldc + u]);
    const float cp = c_prev ? c_prev[(int64_t)b * ldcp + u] : 0.0f;
    float dh = dout_t[(int64_t)b * ldo + u];
    if (dh_rec) for (int p = 0; p < nparts; ++p) dh += dh_rec[(int64_t)p * total + e];   // partials of Wh' * dgates
    const float d_o = dh * tc;
    const float dcc = dc[e] + dh * og * (1.0f - tc * tc);
    gr[u] = dcc * gg * ig * (1.0f - ig);
    gr[H + u] = dcc * cp * fg * (1.0f - fg);
    gr[2 * H + u] = dcc * ig * (1.0f - gg * gg);
    gr[3 * H + u] = d_o * og * (1.0f - og);
    dc[e] = dcc * fg;
  }
}

// -------------------------------------------------------------------------------- GRU forward step ---
// cache row layout per (b, t): [r (H)][z (H)][hc (H)][gh3 (H)]
template <int HU>
__global__ void __launch_bounds__(RT)
gru_fwd_step_kernel(const float* __restrict__ Wh, const float* __restrict__ gx, int64_t ldgx,
                    const float* __restrict__ hprev, int64_t ldh, float* __restrict__ out_t, int64_t ldo,
                    float* __restrict__ cache_t, int64_t ldcache, float* __restrict__ hT, int H, int B) {
  extern __shared__ float sm[];
  const int kp = (H + KC - 1) / KC * KC;
  constexpr int NR = 3 * HU;
  float* Ws = sm;
  float* vs = Ws + NR * kp;
  float* red = vs + BC * HS;
  const int u0 = blockIdx.x * HU;
  stage_w_rows<3, HU>(Ws, kp, Wh, H, u0);
  for (int b0 = 0; b0 < B; b0 += BC) {
    float acc[NR];
    rows_times_vec<NR>(Ws, kp, hprev, ldh, H, b0, B, vs, acc);
    reduce_quarters<NR>(red, acc);
    for (int e = threadIdx.x; e < BC * HU; e += RT) {
      const int bb = e / HU, u = e % HU;
      const int gb = b0 + bb, gu = u0 + u;
      if (gb < B && gu < H) {
        const float* pre = red + bb * (NR + 1);
        const float* gxr = gx + (int64_t)gb * ldgx;   // includes the bias
        const float gh3 = pre[2 * HU + u];
        const float r = 1.0f / (1.0f + expf(-(gxr[gu] + pre[u])));
        const float z = 1.0f / (1.0f + expf(-(gxr[H + gu] + pre[HU + u])));
        const float hc = tanhf(gxr[2 * H + gu] + r * gh3);
        const float hp = hprev ? hprev[(int64_t)gb * ldh + gu] : 0.0f;
        const float hn = (1.0f - z) * hc + z * hp;
        out_t[(int64_t)gb * ldo + gu] = hn;
        if (cache_t) {
          float* cr = cache_t + (int64_t)gb * ldcache;
          cr[gu] = r; cr[H + gu] = z; cr[2 * H + gu] = hc; cr[3 * H + gu] = gh3;
        }
        if (hT) hT[(int64_t)gb * H + gu] = hn;
      }
    }
  }
}

// GRU gate derivatives for step t.  Writes dgx_t = (da1, da2, da3) and dgh_t = (da1, da2, da3*r), and
// dh_direct = dh*z (the part of dh_{t-1} that does not go through Wh).
__global__ void __launch_bounds__(RT)
gru_bwd_gates_kernel(const float* __restrict__ cache_t, int64_t ldcache, const float* __restrict__ hprev, int64_t ldh,
                     const float* __restrict__ dout_t, int64_t ldo, const float* __restrict__ dh_rec, int nparts,
                     const float* __restrict__ dh_add, float* __restrict__ dgx_t, float* __restrict__ dgh_t, int64_t ldd,
                     float* __restrict__ dh_direct, int H, int B) {
  const int64_t total = (int64_t)B * H;
  for (int64_t e = (int64_t)blockIdx.x * RT + threadIdx.x; e < total; e += (int64_t)gridDim.x * RT) {
    const int b = (int)(e / H), u = (int)(e % H);
    const float* cr = cache_t + (int64_t)b * ldcache;
    const float r = cr[u], z = cr[H + u], hc = cr[2 * H + u], gh3 = cr[3 * H + u];
    const float hp = hprev ? hprev[(int64_t)b * ldh + u] : 0.0f;
    float dh = dout_t[(int64_t)b * ldo + u] + (dh_add ? dh_add[e] : 0.0f);
    if (dh_rec) for (int p = 0; p < nparts; ++p) dh += dh_rec[(int64_t)p * total + e];
    const float da3 = dh * (1.0f - z) * (1.0f - hc * hc);
    const float da2 = dh * (hp - hc) * z * (1.0f - z);
    const float da1 = da3 * gh3 * r * (1.0f - r);
    float* x_ = dgx_t + (int64_t)b * ldd;
    float* h_ = dgh_t + (int64_t)b * ldd;
    x_[u] = da1; x_[H + u] = da2; x_[2 * H + u] = da3;
    h_[u] = da1; h_[H + u] = da2; h_[2 * H + u] = da3 * r;
    dh_direct[e] = dh * z;
  }
}


// =============================================================================================
// Fast step kernels (H a multiple of 4 and small enough for shared memory): every global load of a step is a
// 128-bit load issued up front, so a step costs one memory round trip plus the FMA work.
// =============================================================================================

// pre[b][r] = sum_k W[r][k] * hprev[b][k] for the NG*4 gate rows of units [u0, u0+4) and a 64-wide batch chunk.
//   Ws: [NG*4][kp] (kp = H rounded up to 16), hs: [64][kp + 4], red: [4][64][NG*4 + 1].
//   On return red[b * (NR + 1) + r] holds the sums for this chunk.
// Bounded wait on a shared-memory mbarrier phase.
__device__ __forceinline__ bool rnn_mbar_wait(uint32_t bar, uint32_t parity) {
  for (uint32_t it = 0; it < (1u << 22); ++it) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    if (ok) return true;
  }
  return false;
}

// BULK (persistent kernels): h_{t-1} was written by other blocks of this same launch; its rows (H contiguous floats
// each) are brought into shared memory by one cp.async.bulk per row, which reads through L2 and completes on `bar`.
// hs must have been zeroed once (padding columns and rows past the batch are never written).  Returns false when the
// bounded wait for the copies ran out (uniform over the block).
template <int NG, bool BULK = false>
__device__ __forceinline__ bool fast_gate_preacts(const float* __restrict__ Wh, const float* hprev, int64_t ldh,
                                                  int H, int B, int b0, int u0, int kp, float* __restrict__ Ws,
                                                  float* __restrict__ hs, float* __restrict__ red, bool load_w,
                                                  uint32_t bar = 0, uint32_t parity = 0) {
  constexpr int NR = NG * 4;
  const int hs_ld = kp + 4;
  const int k4n = kp >> 2;
  int ok = 1;
  if (BULK && hprev != nullptr && threadIdx.x < 32) {
    const int nrows = (B - b0) < BC ? (B - b0) : BC;
    asm volatile("fence.proxy.async;" ::: "memory");   // h rows were written through the generic proxy
    if (threadIdx.x == 0)
      asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"((uint32_t)(nrows * H * 4)) : "memory");
    __syncwarp();
    for (int r = threadIdx.x; r < nrows; r += 32) {
      const uint32_t dst = (uint32_t)__cvta_generic_to_shared(hs + r * hs_ld);
      const float* src = hprev + (int64_t)(b0 + r) * ldh;
      asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst), "l"(src),
                   "r"((uint32_t)(H * 4)), "r"(bar)
                   : "memory");
    }
  }
  if (load_w) {
    // W[k][g][u0 .. u0+3] is one 16-byte piece of the [H][NG*H] weight memory
    for (int e = threadIdx.x; e < kp * NG; e += RT) {
      const int k = e / NG, g = e % NG;
      float4 w = make_float4(0.f, 0.f, 0.f, 0.f);
      if (k < H) w = __ldg((const float4*)(Wh + (int64_t)k * (NG * H) + g * H + u0));
      Ws[(g * 4 + 0) * kp + k] = w.x;
      Ws[(g * 4 + 1) * kp + k] = w.y;
      Ws[(g * 4 + 2) * kp + k] = w.z;
      Ws[(g * 4 + 3) * kp + k] = w.w;
    }
  }
  if (hprev != nullptr) {
    if (BULK) {
      ok = rnn_mbar_wait(bar, parity) ? 1 : 0;
    } else {
      for (int e = threadIdx.x; e < BC * k4n; e += RT) {
        const int bb = e / k4n, k4 = e % k4n;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (b0 + bb < B && 4 * k4 < H) v = __ldg((const float4*)(hprev + (int64_t)(b0 + bb) * ldh + 4 * k4));
        *(float4*)(hs + bb * hs_ld + 4 * k4) = v;
      }
    }
  }
  if (!__syncthreads_and(ok)) return false;
  const int b = threadIdx.x & (BC - 1), kq = threadIdx.x >> 6;
  float acc[NR];
#pragma unroll
  for (int r = 0; r < NR; ++r) acc[r] = 0.0f;
  if (hprev != nullptr) {
    const int per = k4n >> 2;                       // float4 steps per quarter
    const float4* hrow = (const float4*)(hs + b * hs_ld) + kq * per;
    for (int i = 0; i < per; ++i) {
      const float4 hv = hrow[i];
      const int kbase = (kq * per + i) * 4;
#pragma unroll
      for (int r = 0; r < NR; ++r) {
        const float4 w = *(const float4*)(Ws + r * kp + kbase);
        acc[r] = fmaf(w.x, hv.x, acc[r]);
        acc[r] = fmaf(w.y, hv.y, acc[r]);
        acc[r] = fmaf(w.z, hv.z, acc[r]);
        acc[r] = fmaf(w.w, hv.w, acc[r]);
      }
    }
  }
#pragma unroll
  for (int r = 0; r < NR; ++r) red[(kq * BC + b) * (NR + 1) + r] = acc[r];
  __syncthreads();
  for (int e = threadIdx.x; e < BC * NR; e += RT) {
    const int bb = e / NR, r = e % NR;
    float sum = 0.0f;
#pragma unroll
    for (int q = 0; q < 4; ++q) sum += red[(q * BC + bb) * (NR + 1) + r];
    red[bb * (NR + 1) + r] = sum;
  }
  __syncthreads();
  return true;
}

__global__ void __launch_bounds__(RT)
lstm_fwd_fast_kernel(const float* __restrict__ Wh, const float* __restrict__ gx, int64_t ldgx,
                     const float* __restrict__ hprev, int64_t ldh, const float* __restrict__ cprev, int64_t ldc,
                     float* __restrict__ out_t, int64_t ldo, float* __restrict__ gates_t, int64_t ldg,
                     float* __restrict__ c_t, int64_t ldct, float* __restrict__ hT, float* __restrict__ cT, int H, int B) {
  extern __shared__ __align__(16) float sm[];
  const int kp = (H + 15) & ~15;
  float* Ws = sm;
  float* hs = Ws + 16 * kp;
  float* red = hs + BC * (kp + 4);
  const int u0 = blockIdx.x * 4;
  for (int b0 = 0; b0 < B; b0 += BC) {
    if (b0 > 0) __syncthreads();
    fast_gate_preacts<4>(Wh, hprev, ldh, H, B, b0, u0, kp, Ws, hs, red, b0 == 0);
    const int bb = threadIdx.x >> 2, u = threadIdx.x & 3;     // 64 x 4 (batch, unit) pairs
    const int gb = b0 + bb, gu = u0 + u;
    if (gb < B && gu < H) {
      const float* pre = red + bb * 17;
      const float* gxr = gx + (int64_t)gb * ldgx;
      const float zi = pre[u] + gxr[gu], zf = pre[4 + u] + gxr[H + gu];
      const float zg = pre[8 + u] + gxr[2 * H + gu], zo = pre[12 + u] + gxr[3 * H + gu];
      const float ig = 1.0f / (1.0f + expf(-zi)), fg = 1.0f / (1.0f + expf(-zf));
      const float gg = tanhf(zg), og = 1.0f / (1.0f + expf(-zo));
      const float cp = cprev ? cprev[(int64_t)gb * ldc + gu] : 0.0f;
      const float cn = fg * cp + ig * gg;
      const float hn = og * tanhf(cn);
      out_t[(int64_t)gb * ldo + gu] = hn;
      if (gates_t) {
        float* gr = gates_t + (int64_t)gb * ldg;
        gr[gu] = ig; gr[H + gu] = fg; gr[2 * H + gu] = gg; gr[3 * H + gu] = og;
      }
      c_t[(int64_t)gb * ldct + gu] = cn;
      if (hT) { hT[(int64_t)gb * H + gu] = hn; cT[(int64_t)gb * H + gu] = cn; }
    }
  }
}

__global__ void __launch_bounds__(RT)
gru_fwd_fast_kernel(const float* __restrict__ Wh, const float* __restrict__ gx, int64_t ldgx,
                    const float* __restrict__ hprev, int64_t ldh, float* __restrict__ out_t, int64_t ldo,
                    float* __restrict__ cache_t, int64_t ldcache, float* __restrict__ hT, int H, int B) {
  extern __shared__ __align__(16) float sm[];
  const int kp = (H + 15) & ~15;
  float* Ws = sm;
  float* hs = Ws + 12 * kp;
  float* red = hs + BC * (kp + 4);
  const int u0 = blockIdx.x * 4;
  for (int b0 = 0; b0 < B; b0 += BC) {
    if (b0 > 0) __syncthreads();
    fast_gate_preacts<3>(Wh, hprev, ldh, H, B, b0, u0, kp, Ws, hs, red, b0 == 0);
    const int bb = threadIdx.x >> 2, u = threadIdx.x & 3;
    const int gb = b0 + bb, gu = u0 + u;
    if (gb < B && gu < H) {
      const float* pre = red + bb * 13;
      const float* gxr = gx + (int64_t)gb * ldgx;   // includes the bias
      const float gh3 = pre[8 + u];
      const float r = 1.0f / (1.0f + expf(-(gxr[gu] + pre[u])));
      const float z = 1.0f / (1.0f + expf(-(gxr[H + gu] + pre[4 + u])));
      const float hc = tanhf(gxr[2 * H + gu] + r * gh3);
      const float hp = hprev ? hprev[(int64_t)gb * ldh + gu] : 0.0f;
      const float hn = (1.0f - z) * hc + z * hp;
      out_t[(int64_t)gb * ldo + gu] = hn;
      if (cache_t) {
        float* cr = cache_t + (int64_t)gb * ldcache;
        cr[gu] = r; cr[H + gu] = z; cr[2 * H + gu] = hc; cr[3 * H + gu] = gh3;
      }
      if (hT) hT[(int64_t)gb * H + gu] = hn;
    }
  }
}

// Barrier over all blocks of a cooperative launch (every block is resident, so every block arrives).  `counter` starts
// at 0 for the launch and counts arrivals; generation g is complete when it reaches g * gridDim.x.  The wait is
// bounded: when it runs out the block records `code` in the error word and every caller leaves its time loop.
constexpr unsigned GRID_WAIT_LIMIT = 1u << 22;
__device__ __forceinline__ bool grid_barrier(unsigned* counter, unsigned target, int32_t* dev_err, int32_t code) {
  __syncthreads();
  int ok = 1;
  if (threadIdx.x == 0) {
    __threadfence();
    atomicAdd(counter, 1u);
    unsigned spins = 0;
    for (;;) {
      unsigned seen;
      asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(seen) : "l"(counter) : "memory");
      if (seen >= target) break;
      if (++spins > GRID_WAIT_LIMIT || *(volatile int32_t*)dev_err != 0) {
        atomicCAS(dev_err, 0, code);
        ok = 0;
        break;
      }
    }
    __threadfence();
  }
  return __syncthreads_and(ok) != 0;
}

// The whole forward time loop in one cooperative launch: block u0/4 keeps its 16 rows of Wh in shared memory for all
// T steps; a step reads h_{t-1} (written by all blocks in the previous step), adds the hoisted input projection,
// applies the gates and writes its 4 units of h_t / c_t; a grid barrier separates the steps.
__global__ void __launch_bounds__(RT)
lstm_fwd_persist_kernel(const float* __restrict__ Wh, const float* __restrict__ gx, const float* __restrict__ h0,
                        const float* __restrict__ c0, float* out, float* gates, float* cst, int cached, float* __restrict__ hT,
                        float* __restrict__ cT, int H, int B, int T, unsigned* counter, int32_t* dev_err) {
  extern __shared__ __align__(16) float sm[];
  const int kp = (H + 15) & ~15;
  float* Ws = sm;
  float* hs = Ws + 16 * kp;
  float* red = hs + BC * (kp + 4);
  const int u0 = blockIdx.x * 4;
  const int64_t ldrow = (int64_t)T * H, ldg = (int64_t)T * 4 * H;
  __shared__ __align__(8) uint64_t h_bar;
  const uint32_t bar = (uint32_t)__cvta_generic_to_shared(&h_bar);
  for (int e = threadIdx.x; e < BC * (kp + 4); e += RT) hs[e] = 0.0f;
  if (threadIdx.x == 0) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(1u) : "memory");
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // the zeros precede the async-proxy row copies
  __syncthreads();
  uint32_t loads = 0;   // bulk loads waited for so far: names the barrier phase
  bool alive = true;
  float gxv[4] = {0.f, 0.f, 0.f, 0.f};
  bool have_gx = false;
  for (int t = 0; t < T && alive; ++t) {
    const float* hprev = t == 0 ? h0 : out + (int64_t)(t - 1) * H;
    const int64_t ldh = t == 0 ? H : ldrow;
    const float* cprev;
    float* c_t;
    int64_t ldcp, ldct;
    if (cached) {
      cprev = t == 0 ? c0 : cst + (int64_t)(t - 1) * H;
      ldcp = t == 0 ? H : ldrow;
      c_t = cst + (int64_t)t * H;
      ldct = ldrow;
    } else {
      cprev = t == 0 ? c0 : cst + (int64_t)((t - 1) & 1) * B * H;
      ldcp = H;
      c_t = cst + (int64_t)(t & 1) * B * H;
      ldct = H;
    }
    const float* gx_t = gx + (int64_t)t * 4 * H;
    float* out_t = out + (int64_t)t * H;
    float* gates_t = gates ? gates + (int64_t)t * 4 * H : nullptr;
    const bool lastt = (t == T - 1);
    for (int b0 = 0; b0 < B; b0 += BC) {
      if (b0 > 0) __syncthreads();
      if (!fast_gate_preacts<4, true>(Wh, hprev, ldh, H, B, b0, u0, kp, Ws, hs, red, t == 0 && b0 == 0, bar, loads & 1u)) {
        if (threadIdx.x == 0) atomicCAS(dev_err, 0, 3002);
        alive = false;
        break;
      }
      if (hprev != nullptr) ++loads;
      const int bb = threadIdx.x >> 2, u = threadIdx.x & 3;
      const int gb = b0 + bb, gu = u0 + u;
      if (gb < B && gu < H) {
        const float* pre = red + bb * 17;
        if (!have_gx) {
          const float* gxr = gx_t + (int64_t)gb * ldg;
          gxv[0] = gxr[gu]; gxv[1] = gxr[H + gu]; gxv[2] = gxr[2 * H + gu]; gxv[3] = gxr[3 * H + gu];
        }
        const float zi = pre[u] + gxv[0], zf = pre[4 + u] + gxv[1];
        const float zg = pre[8 + u] + gxv[2], zo = pre[12 + u] + gxv[3];
        const float ig = 1.0f / (1.0f + expf(-zi)), fg = 1.0f / (1.0f + expf(-zf));
        const float gg = tanhf(zg), og = 1.0f / (1.0f + expf(-zo));
        // c of (gb, gu) was written by this same thread one step earlier
        const float cp = cprev ? cprev[(int64_t)gb * ldcp + gu] : 0.0f;
        const float cn = fg * cp + ig * gg;
        const float hn = og * tanhf(cn);
        out_t[(int64_t)gb * ldrow + gu] = hn;
        if (gates_t) {
          float* gr = gates_t + (int64_t)gb * ldg;
          gr[gu] = ig; gr[H + gu] = fg; gr[2 * H + gu] = gg; gr[3 * H + gu] = og;
        }
        c_t[(int64_t)gb * ldct + gu] = cn;
        if (lastt && hT) { hT[(int64_t)gb * H + gu] = hn; cT[(int64_t)gb * H + gu] = cn; }
      }
    }
    // the input projection of the next step does not depend on the recurrence: fetch it while waiting at the barrier
    have_gx = false;
    if (B <= BC && !lastt) {
      const int gb = threadIdx.x >> 2, gu = u0 + (threadIdx.x & 3);
      if (gb < B && gu < H) {
        const float* gxr = gx + (int64_t)(t + 1) * 4 * H + (int64_t)gb * ldg;
        gxv[0] = gxr[gu]; gxv[1] = gxr[H + gu]; gxv[2] = gxr[2 * H + gu]; gxv[3] = gxr[3 * H + gu];
        have_gx = true;
      }
    }
    if (alive && !lastt && !grid_barrier(counter, (unsigned)(t + 1) * gridDim.x, dev_err, 3001)) break;
  }
}

// Register-tiled persistent forward time loop (H and B multiples of 16) for LSTM (NG = 4 gates) and GRU (NG = 3):
// block (unit group, batch group) owns 16 hidden units - their NG * 16 gate rows of Wh, resident in shared memory as
// Ws[k][NG * 16] for all T steps - and 16 batch columns.  A step stages only the 16 rows of h_{t-1} the block needs
// (32 KB at H = 512 instead of all 64 rows), and every thread accumulates a 4-row x 4-column tile over a quarter of k:
// per four k-values 8 shared-memory loads of 16 bytes feed 64 FMAs (the row-per-thread scheme of the *_persist
// kernels issues 17 loads per 64 FMAs and is bound by them).  The four k-quarters are summed through shared memory
// by the thread that owns (unit, column) in the gate stage; for the LSTM that thread also keeps c of the pair in a
// register.  Only the blocks of one batch group exchange h rows, so each group has its own barrier counter.
//   shared memory: Ws [H][NG * 16], hs [16][H + 4], red [4][NG * 16][17]
//   LSTM: cache = gates [rows][4H] (or NULL), cst = cell states, gx [rows][4H].  GRU: cache = (r, z, hc, gh3)
//   [rows][4H] (or NULL), gx [rows][3H]; c0 / cst / cT unused.
constexpr int TU = 16, TB = 16;
inline size_t tile_fwd_smem(int ng, int H) {
  return ((size_t)H * ng * 16 + (size_t)TB * (H + 4) + (size_t)4 * ng * 16 * 17) * sizeof(float);
}

template <int NG>
__global__ void __launch_bounds__(RT, 1)
rnn_fwd_tile_kernel(const float* __restrict__ Wh, const float* __restrict__ gx, const float* __restrict__ h0,
                    const float* __restrict__ c0, float* out, float* cache, float* cst, int cached, float* __restrict__ hT,
                    float* __restrict__ cT, int H, int B, int T, unsigned* counter, int32_t* dev_err) {
  constexpr int NR = NG * 16;
  extern __shared__ __align__(16) float sm[];
  const int hs_ld = H + 4;
  float* Ws = sm;
  float* hs = Ws + (size_t)H * NR;
  float* red = hs + TB * hs_ld;
  const int ugroups = H / TU;
  const int u0 = ((int)blockIdx.x % ugroups) * TU, b0 = ((int)blockIdx.x / ugroups) * TB;
  const int64_t ldrow = (int64_t)T * H, ldgx = (int64_t)T * NG * H, ldc = (int64_t)T * 4 * H;
  __shared__ __align__(8) uint64_t h_bar;
  const uint32_t bar = (uint32_t)__cvta_generic_to_shared(&h_bar);
  if (threadIdx.x == 0) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(1u) : "memory");
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  // Ws[k][g * 16 + u] = Wh[g * H + u0 + u][k]: 16 consecutive floats of the [H][NG * H] weight memory per (k, g)
  for (int e = threadIdx.x; e < H * (NG * 4); e += RT) {
    const int k = e / (NG * 4), q = e % (NG * 4), g = q >> 2, part = q & 3;
    const float4 w = __ldg((const float4*)(Wh + (int64_t)k * (NG * H) + g * H + u0 + part * 4));
    *(float4*)(Ws + (size_t)k * NR + g * 16 + part * 4) = w;
  }
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  __syncthreads();
  const int kq = threadIdx.x >> 6, rg = (threadIdx.x & 63) >> 2, bgi = threadIdx.x & 3;   // tile roles
  const int gu = threadIdx.x & 15, gb = threadIdx.x >> 4;                                 // gate-stage roles
  const int b = b0 + gb, u = u0 + gu;
  const int per = H >> 2;   // k-values per quarter (a multiple of 4)
  uint32_t loads = 0;       // bulk loads waited for so far: names the barrier phase
  float gxv[NG];
  bool have_gx = false;
  // LSTM: the cell state of (column, unit) stays in a register of the thread that owns the pair in the gate stage
  float c_reg = (NG == 4 && c0) ? c0[(int64_t)b * H + u] : 0.0f;
  unsigned* my_counter = counter + (int)blockIdx.x / ugroups;
  for (int t = 0; t < T; ++t) {
    const float* hprev = t == 0 ? h0 : out + (int64_t)(t - 1) * H;
    const int64_t ldh = t == 0 ? H : ldrow;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;
    if (hprev != nullptr) {
      if (threadIdx.x < 32) {
        asm volatile("fence.proxy.async;" ::: "memory");   // h rows were written through the generic proxy
        if (threadIdx.x == 0)
          asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"((uint32_t)(TB * H * 4)) : "memory");
        __syncwarp();
        if (threadIdx.x < TB) {
          const uint32_t dst = (uint32_t)__cvta_generic_to_shared(hs + threadIdx.x * hs_ld);
          const float* src = hprev + (int64_t)(b0 + (int)threadIdx.x) * ldh;
          asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst), "l"(src),
                       "r"((uint32_t)(H * 4)), "r"(bar)
                       : "memory");
        }
      }
      const int ok = rnn_mbar_wait(bar, loads & 1u) ? 1 : 0;
      ++loads;
      if (!__syncthreads_and(ok)) {
        if (threadIdx.x == 0) atomicCAS(dev_err, 0, 3002);
        return;
      }
      if (rg < NG * 4) {
        const float* hbase = hs + bgi * hs_ld;
        const float* wbase = Ws + rg * 4;
        for (int k = kq * per; k < (kq + 1) * per; k += 4) {
          float4 hv[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) hv[j] = *(const float4*)(hbase + (4 * j) * hs_ld + k);   // columns bgi, bgi+4, bgi+8, bgi+12
#pragma unroll
          for (int kk = 0; kk < 4; ++kk) {
            const float4 w = *(const float4*)(wbase + (size_t)(k + kk) * NR);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const float hk = kk == 0 ? hv[j].x : kk == 1 ? hv[j].y : kk == 2 ? hv[j].z : hv[j].w;
              acc[0][j] = fmaf(w.x, hk, acc[0][j]);
              acc[1][j] = fmaf(w.y, hk, acc[1][j]);
              acc[2][j] = fmaf(w.z, hk, acc[2][j]);
              acc[3][j] = fmaf(w.w, hk, acc[3][j]);
            }
          }
        }
      }
    }
    if (rg < NG * 4) {
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) red[(kq * NR + rg * 4 + i) * 17 + bgi + 4 * j] = acc[i][j];
    }
    __syncthreads();
    {
      float pre[NG];
#pragma unroll
      for (int g = 0; g < NG; ++g) {
        float sum = 0.0f;
#pragma unroll
        for (int q = 0; q < 4; ++q) sum += red[(q * NR + g * 16 + gu) * 17 + gb];
        pre[g] = sum;
      }
      if (!have_gx) {
        const float* gxr = gx + (int64_t)t * NG * H + (int64_t)b * ldgx;
#pragma unroll
        for (int g = 0; g < NG; ++g) gxv[g] = gxr[g * H + u];
      }
      float hn;
      if (NG == 4) {
        const float zi = pre[0] + gxv[0], zf = pre[1] + gxv[1], zg = pre[2] + gxv[2], zo = pre[NG - 1] + gxv[NG - 1];
        const float ig = 1.0f / (1.0f + expf(-zi)), fg = 1.0f / (1.0f + expf(-zf));
        const float gg = tanhf(zg), og = 1.0f / (1.0f + expf(-zo));
        const float cn = fg * c_reg + ig * gg;
        c_reg = cn;
        hn = og * tanhf(cn);
        if (cache) {
          float* gr = cache + (int64_t)t * 4 * H + (int64_t)b * ldc;
          gr[u] = ig; gr[H + u] = fg; gr[2 * H + u] = gg; gr[3 * H + u] = og;
        }
        float* c_t = cached ? cst + (int64_t)t * H + (int64_t)b * ldrow : cst + (int64_t)(t & 1) * B * H + (int64_t)b * H;
        c_t[u] = cn;
        if (t == T - 1 && hT) cT[(int64_t)b * H + u] = cn;
      } else {
        const float gh3 = pre[2];
        const float r = 1.0f / (1.0f + expf(-(gxv[0] + pre[0])));
        const float z = 1.0f / (1.0f + expf(-(gxv[1] + pre[1])));
        const float hc = tanhf(gxv[2] + r * gh3);
        const float hp = hprev ? hs[gb * hs_ld + u] : 0.0f;   // the staged row of h_{t-1}
        hn = (1.0f - z) * hc + z * hp;
        if (cache) {
          float* cr = cache + (int64_t)t * 4 * H + (int64_t)b * ldc;
          cr[u] = r; cr[H + u] = z; cr[2 * H + u] = hc; cr[3 * H + u] = gh3;
        }
      }
      out[(int64_t)t * H + (int64_t)b * ldrow + u] = hn;
      if (t == T - 1 && hT) hT[(int64_t)b * H + u] = hn;
      // the input projection of the next step does not depend on the recurrence: fetch it before the barrier
      have_gx = false;
      if (t + 1 < T) {
        const float* gxr = gx + (int64_t)(t + 1) * NG * H + (int64_t)b * ldgx;
#pragma unroll
        for (int g = 0; g < NG; ++g) gxv[g] = gxr[g * H + u];
        have_gx = true;
      }
    }
    if (t + 1 < T && !grid_barrier(my_counter, (unsigned)(t + 1) * (unsigned)ugroups, dev_err, 3001)) break;
  }
}

// GRU counterpart of lstm_fwd_persist_kernel: block u0/4 keeps its 12 rows of Wh in shared memory for all T steps.
__global__ void __launch_bounds__(RT)
gru_fwd_persist_kernel(const float* __restrict__ Wh, const float* __restrict__ gx, const float* __restrict__ h0, float* out,
                       float* cch, float* __restrict__ hT, int H, int B, int T, unsigned* counter, int32_t* dev_err) {
  extern __shared__ __align__(16) float sm[];
  const int kp = (H + 15) & ~15;
  float* Ws = sm;
  float* hs = Ws + 12 * kp;
  float* red = hs + BC * (kp + 4);
  const int u0 = blockIdx.x * 4;
  const int64_t ldrow = (int64_t)T * H, ldgx = (int64_t)T * 3 * H, ldc = (int64_t)T * 4 * H;
  __shared__ __align__(8) uint64_t h_bar;
  const uint32_t bar = (uint32_t)__cvta_generic_to_shared(&h_bar);
  for (int e = threadIdx.x; e < BC * (kp + 4); e += RT) hs[e] = 0.0f;
  if (threadIdx.x == 0) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(1u) : "memory");
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  __syncthreads();
  uint32_t loads = 0;
  bool alive = true;
  for (int t = 0; t < T && alive; ++t) {
    const float* hprev = t == 0 ? h0 : out + (int64_t)(t - 1) * H;
    const int64_t ldh = t == 0 ? H : ldrow;
    const float* gx_t = gx + (int64_t)t * 3 * H;
    float* out_t = out + (int64_t)t * H;
    float* c_t = cch ? cch + (int64_t)t * 4 * H : nullptr;
    const bool lastt = (t == T - 1);
    for (int b0 = 0; b0 < B; b0 += BC) {
      if (b0 > 0) __syncthreads();
      if (!fast_gate_preacts<3, true>(Wh, hprev, ldh, H, B, b0, u0, kp, Ws, hs, red, t == 0 && b0 == 0, bar, loads & 1u)) {
        if (threadIdx.x == 0) atomicCAS(dev_err, 0, 3002);
        alive = false;
        break;
      }
      if (hprev != nullptr) ++loads;
      const int bb = threadIdx.x >> 2, u = threadIdx.x & 3;
      const int gb = b0 + bb, gu = u0 + u;
      if (gb < B && gu < H) {
        const float* pre = red + bb * 13;
        const float* gxr = gx_t + (int64_t)gb * ldgx;   // includes the bias
        const float gh3 = pre[8 + u];
        const float r = 1.0f / (1.0f + expf(-(gxr[gu] + pre[u])));
        const float z = 1.0f / (1.0f + expf(-(gxr[H + gu] + pre[4 + u])));
        const float hc = tanhf(gxr[2 * H + gu] + r * gh3);
        const float hp = hprev ? hs[bb * (kp + 4) + gu] : 0.0f;   // the staged row of h_{t-1}
        const float hn = (1.0f - z) * hc + z * hp;
        out_t[(int64_t)gb * ldrow + gu] = hn;
        if (c_t) {
          float* cr = c_t + (int64_t)gb * ldc;
          cr[gu] = r; cr[H + gu] = z; cr[2 * H + gu] = hc; cr[3 * H + gu] = gh3;
        }
        if (lastt && hT) hT[(int64_t)gb * H + gu] = hn;
      }
    }
    if (alive && !lastt && !grid_barrier(counter, (unsigned)(t + 1) * gridDim.x, dev_err, 3001)) break;
  }
}

size_t fast_fwd_smem(int ng, int H) {
  const int kp = (H + 15) & ~15;
  return (size_t)(ng * 4 * kp + BC * (kp + 4) + 4 * BC * (ng * 4 + 1)) * sizeof(float);
}

// dh partials, 2-d decomposition: block (ub, rb, bz) computes, for units [64 ub, +64) and batch rows [64 bz, +64),
// the partial sum over gate rows r in [256 rb, +256):  part[rb][b][u] = sum_r dg[b][r] * Wm[u][r].
// Wm is the weight memory [H][R] (rows of R contiguous floats), so both operands stream as 128-bit loads.
constexpr int DH_U = 64, DH_R = 256, DH_LD = DH_R + 4;

__global__ void __launch_bounds__(RT)
rnn_bwd_dh2d_kernel(const float* __restrict__ Wh, const float* __restrict__ dg, int64_t ldg, float* __restrict__ part,
                    int H, int R, int B) {
  extern __shared__ __align__(16) float sm[];
  float* Ws = sm;                   // [64 u][DH_LD]
  float* Ds = Ws + DH_U * DH_LD;    // [64 b][DH_LD]
  const int u0 = blockIdx.x * DH_U, r0 = blockIdx.y * DH_R, b0 = blockIdx.z * BC;
  const bool vec = ((R & 3) == 0) && ((ldg & 3) == 0) && ((((uintptr_t)Wh | (uintptr_t)dg) & 15) == 0);
  for (int e = threadIdx.x; e < DH_U * (DH_R / 4); e += RT) {
    const int row = e / (DH_R / 4), c4 = e % (DH_R / 4);
    const int r = r0 + 4 * c4;
    float4 w = make_float4(0.f, 0.f, 0.f, 0.f), d = make_float4(0.f, 0.f, 0.f, 0.f);
    if (vec && r + 3 < R) {
      if (u0 + row < H) w = __ldg((const float4*)(Wh + (int64_t)(u0 + row) * R + r));
      if (b0 + row < B) d = __ldg((const float4*)(dg + (int64_t)(b0 + row) * ldg + r));
    } else {
      float wv[4] = {0.f, 0.f, 0.f, 0.f}, dv[4] = {0.f, 0.f, 0.f, 0.f};
      for (int i = 0; i < 4; ++i)
        if (r + i < R) {
          if (u0 + row < H) wv[i] = Wh[(int64_t)(u0 + row) * R + r + i];
          if (b0 + row < B) dv[i] = dg[(int64_t)(b0 + row) * ldg + r + i];
        }
      w = make_float4(wv[0], wv[1], wv[2], wv[3]);
      d = make_float4(dv[0], dv[1], dv[2], dv[3]);
    }
    *(float4*)(Ws + row * DH_LD + 4 * c4) = w;
    *(float4*)(Ds + row * DH_LD + 4 * c4) = d;
  }
  __syncthreads();
  // 16 x 16 threads, each a 4 x 4 tile: rows b = ty + 16 i, columns u = tx + 16 j
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;
  for (int c = 0; c < DH_R; c += 4) {
    float4 a[4], b[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) a[i] = *(const float4*)(Ds + (ty + 16 * i) * DH_LD + c);
#pragma unroll
    for (int j = 0; j < 4; ++j) b[j] = *(const float4*)(Ws + (tx + 16 * j) * DH_LD + c);
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        acc[i][j] = fmaf(a[i].x, b[j].x, acc[i][j]);
        acc[i][j] = fmaf(a[i].y, b[j].y, acc[i][j]);
        acc[i][j] = fmaf(a[i].z, b[j].z, acc[i][j]);
        acc[i][j] = fmaf(a[i].w, b[j].w, acc[i][j]);
      }
  }
  float* pp = part + (int64_t)blockIdx.y * B * H;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int gb = b0 + ty + 16 * i;
    if (gb >= B) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int gu = u0 + tx + 16 * j;
      if (gu < H) pp[(int64_t)gb * H + gu] = acc[i][j];
    }
  }
}

constexpr size_t DH2D_SMEM = (size_t)2 * DH_U * DH_LD * sizeof(float);

// The whole LSTM reverse time loop in one cooperative launch.  Block (ub, rb, bz) keeps the 64 x 128 tile
// Wm[64 ub .. +64][128 rb .. +128] of the recurrent weights in shared memory for all T steps.  A step has two phases
// separated by grid barriers: (1) every thread turns its (b, u) elements' dh = dout + sum of the partials of the step
// after into the four gate derivatives (written over the cached gates) and carries dc; (2) every block multiplies
// its weight tile with its 64 x 128 tile of those derivatives into the partial sums
// part[rb][b][u] that phase 1 of the next step adds up.
constexpr int PB_R = 128, PB_LD = PB_R + 4;
constexpr size_t PB_SMEM = (size_t)2 * DH_U * PB_LD * sizeof(float);

__global__ void __launch_bounds__(RT)
lstm_bwd_persist_kernel(const float* __restrict__ Wh, float* gates, const float* __restrict__ cst, const float* __restrict__ c0,
                        const float* __restrict__ dout, const float* __restrict__ dhT, float* dc, float* parts, int H, int B, int T,
                        int UB, int NP, unsigned* counter, int32_t* dev_err) {
  extern __shared__ __align__(16) float sm[];
  float* Ws = sm;                   // [64 u][PB_LD]
  float* Ds = Ws + DH_U * PB_LD;    // [64 b][PB_LD]
  const int R = 4 * H;
  const int ub = blockIdx.x % UB, rb = (blockIdx.x / UB) % NP, bz = blockIdx.x / (UB * NP);
  const int u0 = ub * DH_U, r0 = rb * PB_R, b0 = bz * BC;
  const int64_t ldrow = (int64_t)T * H, ldg = (int64_t)T * 4 * H, total = (int64_t)B * H;
  for (int e = threadIdx.x; e < DH_U * (PB_R / 4); e += RT) {
    const int row = e / (PB_R / 4), c4 = e % (PB_R / 4);
    float4 w = make_float4(0.f, 0.f, 0.f, 0.f);
    if (u0 + row < H) w = __ldg((const float4*)(Wh + (int64_t)(u0 + row) * R + r0 + 4 * c4));
    *(float4*)(Ws + row * PB_LD + 4 * c4) = w;
    *(float4*)(Ds + row * PB_LD + 4 * c4) = make_float4(0.f, 0.f, 0.f, 0.f);
  }
  __syncthreads();
  const int nrows = (B - b0) < BC ? (B - b0) : BC;
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  unsigned gen = 0;      // grid barriers passed
  for (int t = T - 1; t >= 0; --t) {
    // ---- phase 1: gate derivatives of step t
    {
      float* g_t = gates + (int64_t)t * 4 * H;
      const float* c_t = cst + (int64_t)t * H;
      const float* c_prev = t == 0 ? c0 : cst + (int64_t)(t - 1) * H;
      const int64_t ldcp = t == 0 ? (int64_t)H : ldrow;
      const float* dout_t = dout + (int64_t)t * H;
      const bool lastt = (t == T - 1);
      for (int64_t e = (int64_t)blockIdx.x * RT + threadIdx.x; e < total; e += (int64_t)gridDim.x * RT) {
        const int b = (int)(e / H), u = (int)(e % H);
        float* gr = g_t + (int64_t)b * ldg;
        const float ig = gr[u], fg = gr[H + u], gg = gr[2 * H + u], og = gr[3 * H + u];
        const float tc = tanhf(c_t[(int64_t)b * ldrow + u]);
        const float cp = c_prev ? c_prev[(int64_t)b * ldcp + u] : 0.0f;
        float dh = dout_t[(int64_t)b * ldrow + u];
        if (lastt) {
          if (dhT) dh += dhT[e];
        } else {
          // partials written by other blocks: four loads in flight at a time, added in a fixed order
          const float* pe = parts + e;
          int p = 0;
          for (; p + 4 <= NP; p += 4) {
            const float q0 = __ldcg(pe + (int64_t)p * total), q1 = __ldcg(pe + (int64_t)(p + 1) * total);
            const float q2 = __ldcg(pe + (int64_t)(p + 2) * total), q3 = __ldcg(pe + (int64_t)(p + 3) * total);
            dh += (q0 + q1) + (q2 + q3);
          }
          for (; p < NP; ++p) dh += __ldcg(pe + (int64_t)p * total);
        }
        const float d_o = dh * tc;
        const float dcc = dc[e] + dh * og * (1.0f - tc * tc);   // dc[e] is carried by this same thread
        gr[u] = dcc * gg * ig * (1.0f - ig);
        gr[H + u] = dcc * cp * fg * (1.0f - fg);
        gr[2 * H + u] = dcc * ig * (1.0f - gg * gg);
        gr[3 * H + u] = d_o * og * (1.0f - og);
        dc[e] = dcc * fg;
      }
    }
    if (t == 0) break;
    ++gen;
    if (!grid_barrier(counter, gen * gridDim.x, dev_err, 3003)) break;
    // ---- phase 2: partial sums of Wh' * dgates for step t - 1
    {
      // the 64 x 128 tile of derivatives (written by other blocks: read through L2), eight 128-bit loads in flight
      // per thread
      constexpr int PER = DH_U * (PB_R / 4) / RT;   // 8
      float4 v[PER];
      const float* base = gates + (int64_t)t * 4 * H + r0;
#pragma unroll
      for (int i = 0; i < PER; ++i) {
        const int e = threadIdx.x + i * RT;
        const int row = e / (PB_R / 4), c4 = e % (PB_R / 4);
        v[i] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (row < nrows) v[i] = __ldcg((const float4*)(base + (int64_t)(b0 + row) * ldg + 4 * c4));
      }
#pragma unroll
      for (int i = 0; i < PER; ++i) {
        const int e = threadIdx.x + i * RT;
        const int row = e / (PB_R / 4), c4 = e % (PB_R / 4);
        *(float4*)(Ds + row * PB_LD + 4 * c4) = v[i];
      }
      __syncthreads();
    }
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;
#pragma unroll 4
    for (int c = 0; c < PB_R; c += 4) {
      float4 a[4], w[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = *(const float4*)(Ds + (ty + 16 * i) * PB_LD + c);
#pragma unroll
      for (int j = 0; j < 4; ++j) w[j] = *(const float4*)(Ws + (tx + 16 * j) * PB_LD + c);
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          acc[i][j] = fmaf(a[i].x, w[j].x, acc[i][j]);
          acc[i][j] = fmaf(a[i].y, w[j].y, acc[i][j]);
          acc[i][j] = fmaf(a[i].z, w[j].z, acc[i][j]);
          acc[i][j] = fmaf(a[i].w, w[j].w, acc[i][j]);
        }
    }
    float* pp = parts + (int64_t)rb * total;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int gb = b0 + ty + 16 * i;
      if (gb >= B) continue;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int gu = u0 + tx + 16 * j;
        if (gu < H) pp[(int64_t)gb * H + gu] = acc[i][j];
      }
    }
    ++gen;
    if (!grid_barrier(counter, gen * gridDim.x, dev_err, 3003)) break;
  }
}


// hprev_all[(b, t)] = t == 0 ? h0[b] (or 0) : out[(b, t-1)]
__global__ void __launch_bounds__(RT)
shift_prev_kernel(const float* __restrict__ out, const float* __restrict__ h0, float* __restrict__ hprev_all, int H,
                  int64_t T, int64_t B) {
  const int64_t total = B * T * H;
  for (int64_t e = (int64_t)blockIdx.x * RT + threadIdx.x; e < total; e += (int64_t)gridDim.x * RT) {
    const int64_t row = e / H;
    const int u = (int)(e % H);
    const int64_t t = row % T, b = row / T;
    hprev_all[e] = t == 0 ? (h0 ? h0[b * H + u] : 0.0f) : out[e - H];
  }
}

// db[j] = sum over rows of dg[row][j]
int32_t colsum_rows(fb_ctx* ctx, cudaStream_t stream, const float* dg, float* db, int64_t rows, int64_t cols) {
  return fb_act_bwd_colsum(ctx, stream, FB_ACT_IDENTITY, dg, nullptr, nullptr, nullptr, db, rows, cols);
}

int pick_hu(int ng, int H, size_t smem_optin, size_t extra) {
  const int kp = (H + KC - 1) / KC * KC;
  const int cand[3] = {4, 2, 1};
  for (int i = 0; i < 3; ++i) {
    const size_t need = (size_t)(ng * cand[i]) * kp * 4 + extra + (size_t)4 * BC * (ng * cand[i] + 1) * 4;
    if (need <= smem_optin) return cand[i];
  }
  return 0;
}

size_t fwd_smem(int ng, int hu, int H) {
  const int kp = (H + KC - 1) / KC * KC;
  return (size_t)(ng * hu) * kp * 4 + (size_t)BC * HS * 4 + (size_t)4 * BC * (ng * hu + 1) * 4;
}

// FLUXB200_RNN_PERSIST = 0 keeps one launch per time step.
bool persistent_enabled() {
  static int on = -1;
  if (on < 0) {
    const char* e = getenv("FLUXB200_RNN_PERSIST");
    on = (e != nullptr && e[0] == '0') ? 0 : 1;
  }
  return on != 0;
}

// The persistent kernels synchronise their blocks with a bounded barrier of their own, which needs every block
// resident at once.  Outside a stream capture they are launched cooperatively (the runtime then guarantees it, or
// refuses).  A cooperative launch cannot be recorded into a CUDA graph, so under capture the same kernel is launched
// plainly: its grid was sized by the occupancy query to fit the GPU, and a replayed graph starts it when the stream's
// previous kernel has ended; should another stream hold SMs at that moment, the barrier's limit ends the launch with
// code 3001-3004 in the device error word instead of waiting for ever.
// GRU counterpart of lstm_bwd_persist_kernel: the whole reverse time loop in one cooperative launch.  Phase 1 of step t
// forms the gate derivatives (dgx_t, dgh_t) from dh = dout_t + dh_direct + the partial sums of the step after it;
// phase 2 lets block (ub, rb, bz) multiply its resident 64 x 128 tile of Wh with the 64 x 128 tile of dgh_t into
// partial sums of dh_{t-1}.  dh_direct (dh * z) is carried by the thread that wrote it.  R = 3H need not be a multiple
// of 128: columns past R are zero in both tiles.
__global__ void __launch_bounds__(RT, 1)
gru_bwd_persist_kernel(const float* __restrict__ Wh, const float* __restrict__ cch, const float* __restrict__ out,
                       const float* __restrict__ h0, const float* __restrict__ dout, const float* __restrict__ dhT, float* dgx,
                       float* dgh, float* dh_direct, float* parts, int H, int B, int T, int UB, int NP, unsigned* counter,
                       int32_t* dev_err) {
  extern __shared__ __align__(16) float sm[];
  float* Ws = sm;                   // [64 u][PB_LD]
  float* Ds = Ws + DH_U * PB_LD;    // [64 b][PB_LD]
  const int R = 3 * H;
  const int ub = blockIdx.x % UB, rb = (blockIdx.x / UB) % NP, bz = blockIdx.x / (UB * NP);
  const int u0 = ub * DH_U, r0 = rb * PB_R, b0 = bz * BC;
  const int64_t ldrow = (int64_t)T * H, ldc = (int64_t)T * 4 * H, ldd = (int64_t)T * 3 * H, total = (int64_t)B * H;
  for (int e = threadIdx.x; e < DH_U * (PB_R / 4); e += RT) {
    const int row = e / (PB_R / 4), c4 = e % (PB_R / 4);
    float4 w = make_float4(0.f, 0.f, 0.f, 0.f);
    if (u0 + row < H && r0 + 4 * c4 < R) w = __ldg((const float4*)(Wh + (int64_t)(u0 + row) * R + r0 + 4 * c4));
    *(float4*)(Ws + row * PB_LD + 4 * c4) = w;
    *(float4*)(Ds + row * PB_LD + 4 * c4) = make_float4(0.f, 0.f, 0.f, 0.f);
  }
  __syncthreads();
  const int nrows = (B - b0) < BC ? (B - b0) : BC;
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  unsigned gen = 0;      // grid barriers passed
  for (int t = T - 1; t >= 0; --t) {
    // ---- phase 1: gate derivatives of step t
    {
      const float* c_t = cch + (int64_t)t * 4 * H;
      const float* dout_t = dout + (int64_t)t * H;
      float* dgx_t = dgx + (int64_t)t * 3 * H;
      float* dgh_t = dgh + (int64_t)t * 3 * H;
      const bool lastt = (t == T - 1);
      for (int64_t e = (int64_t)blockIdx.x * RT + threadIdx.x; e < total; e += (int64_t)gridDim.x * RT) {
        const int b = (int)(e / H), u = (int)(e % H);
        const float* cr = c_t + (int64_t)b * ldc;
        const float r = cr[u], z = cr[H + u], hc = cr[2 * H + u], gh3 = cr[3 * H + u];
        const float hp = t == 0 ? (h0 ? h0[e] : 0.0f) : out[(int64_t)(t - 1) * H + (int64_t)b * ldrow + u];
        float dh = dout_t[(int64_t)b * ldrow + u];
        if (lastt) {
          if (dhT) dh += dhT[e];
        } else {
          dh += dh_direct[e];   // written by this same thread one step earlier
          // partials written by other blocks: four loads in flight at a time, added in a fixed order
          const float* pe = parts + e;
          int p = 0;
          for (; p + 4 <= NP; p += 4) {
            const float q0 = __ldcg(pe + (int64_t)p * total), q1 = __ldcg(pe + (int64_t)(p + 1) * total);
            const float q2 = __ldcg(pe + (int64_t)(p + 2) * total), q3 = __ldcg(pe + (int64_t)(p + 3) * total);
            dh += (q0 + q1) + (q2 + q3);
          }
          for (; p < NP; ++p) dh += __ldcg(pe + (int64_t)p * total);
        }
        const float da3 = dh * (1.0f - z) * (1.0f - hc * hc);
        const float da2 = dh * (hp - hc) * z * (1.0f - z);
        const float da1 = da3 * gh3 * r * (1.0f - r);
        float* x_ = dgx_t + (int64_t)b * ldd;
        float* h_ = dgh_t + (int64_t)b * ldd;
        x_[u] = da1; x_[H + u] = da2; x_[2 * H + u] = da3;
        h_[u] = da1; h_[H + u] = da2; h_[2 * H + u] = da3 * r;
        dh_direct[e] = dh * z;
      }
    }
    if (t == 0) break;
    ++gen;
    if (!grid_barrier(counter, gen * gridDim.x, dev_err, 3004)) break;
    // ---- phase 2: partial sums of Wh' * dgh_t (the recurrent part of dh_{t-1})
    {
      constexpr int PER = DH_U * (PB_R / 4) / RT;   // 8
      float4 v[PER];
      const float* base = dgh + (int64_t)t * 3 * H + r0;
#pragma unroll
      for (int i = 0; i < PER; ++i) {
        const int e = threadIdx.x + i * RT;
        const int row = e / (PB_R / 4), c4 = e % (PB_R / 4);
        v[i] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (row < nrows && r0 + 4 * c4 < R) v[i] = __ldcg((const float4*)(base + (int64_t)(b0 + row) * ldd + 4 * c4));
      }
#pragma unroll
      for (int i = 0; i < PER; ++i) {
        const int e = threadIdx.x + i * RT;
        const int row = e / (PB_R / 4), c4 = e % (PB_R / 4);
        *(float4*)(Ds + row * PB_LD + 4 * c4) = v[i];
      }
      __syncthreads();
    }
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;
#pragma unroll 4
    for (int c = 0; c < PB_R; c += 4) {
      float4 a[4], w[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = *(const float4*)(Ds + (ty + 16 * i) * PB_LD + c);
#pragma unroll
      for (int j = 0; j < 4; ++j) w[j] = *(const float4*)(Ws + (tx + 16 * j) * PB_LD + c);
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          acc[i][j] = fmaf(a[i].x, w[j].x, acc[i][j]);
          acc[i][j] = fmaf(a[i].y, w[j].y, acc[i][j]);
          acc[i][j] = fmaf(a[i].z, w[j].z, acc[i][j]);
          acc[i][j] = fmaf(a[i].w, w[j].w, acc[i][j]);
        }
    }
    float* pp = parts + (int64_t)rb * total;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int gb = b0 + ty + 16 * i;
      if (gb >= B) continue;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int gu = u0 + tx + 16 * j;
        if (gu < H) pp[(int64_t)gb * H + gu] = acc[i][j];
      }
    }
    ++gen;
    if (!grid_barrier(counter, gen * gridDim.x, dev_err, 3004)) break;
  }
}

bool persistent_allowed(cudaStream_t) { return persistent_enabled(); }

cudaError_t launch_persistent(const void* kern, dim3 grid, dim3 block, void** args, size_t smem, cudaStream_t stream) {
  cudaStreamCaptureStatus cs = cudaStreamCaptureStatusNone;
  if (cudaStreamIsCapturing(stream, &cs) != cudaSuccess) {
    cudaGetLastError();
    cs = cudaStreamCaptureStatusNone;
  }
  if (cs == cudaStreamCaptureStatusNone) return cudaLaunchCooperativeKernel(kern, grid, block, args, smem, stream);
  return cudaLaunchKernel(kern, grid, block, args, smem, stream);
}

int32_t check_dims(const char* fn, int64_t in_dim, int64_t H, int64_t T, int64_t B) {
  FB_REQUIRE(in_dim >= 1 && H >= 1 && T >= 0 && B >= 0, FB_ERR_SHAPE, "%s: bad shape in=%lld H=%lld T=%lld B=%lld", fn,
             (long long)in_dim, (long long)H, (long long)T, (long long)B);
  FB_REQUIRE(H <= 16384 && B <= (1 << 24) && T <= (1 << 24), FB_ERR_SHAPE, "%s: dimension too large", fn);
  return FB_OK;
}

}  // namespace

FB_API int64_t fb_lstm_cache_bytes(int64_t in_dim, int64_t hidden, int64_t seq_len, int64_t batch) {
  (void)in_dim;
  // gates [B*T][4H] + cell states [B*T][H] + input projection [B*T][4H] (reused as scratch by the backward pass)
  return (int64_t)sizeof(float) * seq_len * batch * hidden * 9;
}

FB_API int64_t fb_gru_cache_bytes(int64_t in_dim, int64_t hidden, int64_t seq_len, int64_t batch) {
  (void)in_dim;
  // (r, z, hc, gh3) [B*T][4H] + input projection [B*T][3H] + recurrent-side gate derivatives [B*T][3H]
  // + shifted hidden states [B*T][H]
  return (int64_t)sizeof(float) * seq_len * batch * hidden * 11;
}

FB_API int32_t fb_lstm_fwd(fb_ctx* ctx, void* stream_, const float* Wi, const float* Wh, const float* b, const float* x,
                           const float* h0, const float* c0, float* out, float* hT, float* cT, void* cache,
                           int64_t in_dim, int64_t hidden, int64_t seq_len, int64_t batch) {
  FB_CHECK_CTX(ctx);
  cudaStream_t stream = (cudaStream_t)stream_;
  int32_t st = check_dims("fb_lstm_fwd", in_dim, hidden, seq_len, batch);
  if (st != FB_OK) return st;
  if (seq_len == 0 || batch == 0) return FB_OK;
  FB_REQUIRE(Wi && Wh && x && out, FB_ERR_INVALID_ARG, "fb_lstm_fwd: NULL pointer");
  FB_REQUIRE((hT == nullptr) == (cT == nullptr), FB_ERR_INVALID_ARG, "fb_lstm_fwd: hT and cT must both be given or both NULL");
  const int H = (int)hidden, B = (int)batch;
  const int64_t T = seq_len, rows = T * batch;
  float *gates, *cst, *gx;
  if (cache) {
    gates = (float*)cache;
    cst = gates + rows * 4 * H;
    gx = cst + rows * H;
  } else {
    float* ws = (float*)fb_scratch(ctx, stream, (size_t)(rows * 4 * H + 2 * (int64_t)B * H) * sizeof(float));
    if (!ws) return FB_ERR_ALLOC;
    gates = nullptr;
    gx = ws;
    cst = ws + rows * 4 * H;   // two [B][H] ping-pong cell buffers
  }
  // (1) input projection for every (b, t): gx[rows][4H] = x[rows][in] * Wi' + b
  fb_gemm_args a;
  a.A = x; a.lda = in_dim; a.a_mn_major = 0;
  a.B = Wi; a.ldb = 4 * hidden; a.b_mn_major = 1;
  a.C = gx; a.ldc = 4 * hidden; a.Z = nullptr; a.bias_n = b; a.bias_m = nullptr;
  a.M = rows; a.N = 4 * hidden; a.K = in_dim; a.act = FB_ACT_IDENTITY; a.accumulate = 0;
  st = fb_gemm_dispatch(ctx, stream, a, FB_PREC_DEFAULT);
  if (st != FB_OK) return st;
  // (2) time loop
  const bool fast = (H % 4 == 0) && fb_aligned16(Wh) && fb_aligned16(out) && (!h0 || fb_aligned16(h0)) &&
                    fast_fwd_smem(4, H) <= ctx->smem_optin;
  const int hu = fast ? 4 : pick_hu(4, H, ctx->smem_optin, (size_t)BC * HS * 4);
  FB_REQUIRE(hu > 0, FB_ERR_UNSUPPORTED, "fb_lstm_fwd: hidden size %d does not fit the step kernel's shared memory", H);
  const size_t smem = fast ? fast_fwd_smem(4, H) : fwd_smem(4, hu, H);
  auto kern = hu == 4 ? lstm_fwd_step_kernel<4> : hu == 2 ? lstm_fwd_step_kernel<2> : lstm_fwd_step_kernel<1>;
  if (fast) FB_CUDA(cudaFuncSetAttribute(lstm_fwd_fast_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  else FB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  const unsigned grid = (unsigned)((H + hu - 1) / hu);
  const int64_t ldrow = T * H;       // stride between batch rows of out / cached c at a fixed t
  if (fast && T > 1 && H % TU == 0 && B % TB == 0 && tile_fwd_smem(4, H) <= ctx->smem_optin && persistent_allowed(stream)) {
    // register-tiled persistent kernel: (H / 16) x (B / 16) blocks, all resident, one cooperative launch
    const int64_t tgrid = (int64_t)(H / TU) * (B / TB);
    const size_t tsmem = tile_fwd_smem(4, H);
    int per_sm = 0;
    FB_CUDA(cudaFuncSetAttribute(rnn_fwd_tile_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)tsmem));
    FB_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, rnn_fwd_tile_kernel<4>, RT, tsmem));
    if ((int64_t)per_sm * ctx->sm_count >= tgrid && T * tgrid < 0x7fffffff && B / TB <= 32) {
      unsigned* counter = (unsigned*)(ctx->dev_error + 16);      // one counter per batch group (at most 32)
      FB_CUDA(cudaMemsetAsync(counter, 0, (size_t)(B / TB) * sizeof(unsigned), stream));
      int cached = cache ? 1 : 0, Hi = H, Bi = B, Ti = (int)T;
      int32_t* dev_err = ctx->dev_error;
      void* args[] = {(void*)&Wh, (void*)&gx, (void*)&h0, (void*)&c0, (void*)&out, (void*)&gates, (void*)&cst, (void*)&cached,
                      (void*)&hT, (void*)&cT, (void*)&Hi, (void*)&Bi, (void*)&Ti, (void*)&counter, (void*)&dev_err};
      FB_CUDA(launch_persistent((const void*)rnn_fwd_tile_kernel<4>, dim3((unsigned)tgrid), dim3(RT), args, tsmem, stream));
      FB_LAUNCH_CHECK();
      return FB_OK;
    }
  }
  if (fast && T > 1 && T * (int64_t)grid < 0x7fffffff && persistent_allowed(stream)) {
    // one cooperative launch for the whole sequence when every block can be resident at once
    int per_sm = 0;
    FB_CUDA(cudaFuncSetAttribute(lstm_fwd_persist_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    FB_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, lstm_fwd_persist_kernel, RT, smem));
    if ((int64_t)per_sm * ctx->sm_count >= (int64_t)grid) {
      unsigned* counter = (unsigned*)(ctx->dev_error + 16);
      FB_CUDA(cudaMemsetAsync(counter, 0, sizeof(unsigned), stream));
      int cached = cache ? 1 : 0, Hi = H, Bi = B, Ti = (int)T;
      int32_t* dev_err = ctx->dev_error;
      void* args[] = {(void*)&Wh, (void*)&gx, (void*)&h0, (void*)&c0, (void*)&out, (void*)&gates, (void*)&cst, (void*)&cached,
                      (void*)&hT, (void*)&cT, (void*)&Hi, (void*)&Bi, (void*)&Ti, (void*)&counter, (void*)&dev_err};
      FB_CUDA(launch_persistent((const void*)lstm_fwd_persist_kernel, dim3(grid), dim3(RT), args, smem, stream));
      FB_LAUNCH_CHECK();
      return FB_OK;
    }
  }
  for (int64_t t = 0; t < T; ++t) {
    const float* hprev = t == 0 ? h0 : out + (t - 1) * H;
    const int64_t ldh = t == 0 ? H : ldrow;
    const float* cprev;
    int64_t ldcp;
    float* c_t;
    int64_t ldct;
    if (cache) {
      cprev = t == 0 ? c0 : cst + (t - 1) * H;
      ldcp = t == 0 ? H : ldrow;
      c_t = cst + t * H;
      ldct = ldrow;
    } else {
      cprev = t == 0 ? c0 : cst + ((t - 1) & 1) * (int64_t)B * H;
      ldcp = H;
      c_t = cst + (t & 1) * (int64_t)B * H;
      ldct = H;
    }
    float* g_t = gates ? gates + t * 4 * H : nullptr;
    float* hT_t = (t == T - 1) ? hT : nullptr;
    float* cT_t = (t == T - 1) ? cT : nullptr;
    if (fast)
      lstm_fwd_fast_kernel<<<grid, RT, smem, stream>>>(Wh, gx + t * 4 * H, T * 4 * H, hprev, ldh, cprev, ldcp, out + t * H, ldrow,
                                                       g_t, T * 4 * H, c_t, ldct, hT_t, cT_t, H, B);
    else
      kern<<<grid, RT, smem, stream>>>(Wh, gx + t * 4 * H, hprev, ldh, cprev, ldcp, out + t * H, ldrow, g_t, c_t, T * 4 * H, ldct,
                                       hT_t, cT_t, H, B, T * 4 * H);
    FB_LAUNCH_CHECK();
  }
  return FB_OK;
}

FB_API int32_t fb_lstm_bwd(fb_ctx* ctx, void* stream_, const float* Wi, const float* Wh, const float* x,
                           const float* h0, const float* c0, const float* out, const void* cache, const float* dout,
                           const float* dhT, const float* dcT,
                           float* dWi, float* dWh, float* db, float* dx, int64_t in_dim, int64_t hidden,
                           int64_t seq_len, int64_t batch) {
  FB_CHECK_CTX(ctx);
  cudaStream_t stream = (cudaStream_t)stream_;
  int32_t st = check_dims("fb_lstm_bwd", in_dim, hidden, seq_len, batch);
  if (st != FB_OK) return st;
  FB_REQUIRE(seq_len >= 1 && batch >= 1, FB_ERR_SHAPE, "fb_lstm_bwd: empty sequence or batch");
  FB_REQUIRE(Wi && Wh && x && out && cache && dout && dWi && dWh, FB_ERR_INVALID_ARG, "fb_lstm_bwd: NULL pointer");
  const int H = (int)hidden, B = (int)batch;
  const int64_t T = seq_len, rows = T * batch, ldrow = T * H;
  float* gates = (float*)cache;              // overwritten in place by the gate derivatives
  const float* cst = gates + rows * 4 * H;
  const int R = 4 * H;
  // one cooperative launch for the whole reverse time loop when its grid can be resident at once
  const int UBp = (H + DH_U - 1) / DH_U, NPp = R / PB_R, BZp = (B + BC - 1) / BC;
  const int64_t pgrid = (int64_t)UBp * NPp * BZp;
  bool persist = T > 1 && (H % 32 == 0) && fb_aligned16(Wh) && fb_aligned16(cache) && pgrid >= 1 && pgrid <= 4096 &&
                 2 * T * pgrid < 0x7fffffff && persistent_allowed(stream);
  if (persist) {
    int per_sm = 0;
    FB_CUDA(cudaFuncSetAttribute(lstm_bwd_persist_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)PB_SMEM));
    FB_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, lstm_bwd_persist_kernel, RT, PB_SMEM));
    persist = (int64_t)per_sm * ctx->sm_count >= pgrid;
  }
  const int nparts = persist ? NPp : (R + DH_R - 1) / DH_R;
  float* ws = (float*)fb_scratch(ctx, stream, (size_t)((1 + nparts) * (int64_t)B * H) * sizeof(float));
  if (!ws) return FB_ERR_ALLOC;
  float* dc = ws;                            // [B][H]
  float* parts = ws + (int64_t)B * H;        // [nparts][B][H] partial sums of Wh' * dgates
  if (dcT) FB_CUDA(cudaMemcpyAsync(dc, dcT, (size_t)B * H * sizeof(float), cudaMemcpyDeviceToDevice, stream));
  else FB_CUDA(cudaMemsetAsync(dc, 0, (size_t)B * H * sizeof(float), stream));
  if (persist) {
    unsigned* counter = (unsigned*)(ctx->dev_error + 16);
    FB_CUDA(cudaMemsetAsync(counter, 0, sizeof(unsigned), stream));
    int Hi = H, Bi = B, Ti = (int)T, ubi = UBp, npi = NPp;
    int32_t* dev_err = ctx->dev_error;
    void* args[] = {(void*)&Wh, (void*)&gates, (void*)&cst, (void*)&c0, (void*)&dout, (void*)&dhT, (void*)&dc, (void*)&parts,
                    (void*)&Hi, (void*)&Bi, (void*)&Ti, (void*)&ubi, (void*)&npi, (void*)&counter, (void*)&dev_err};
    FB_CUDA(launch_persistent((const void*)lstm_bwd_persist_kernel, dim3((unsigned)pgrid), dim3(RT), args, PB_SMEM, stream));
    FB_LAUNCH_CHECK();
  }
  FB_CUDA(cudaFuncSetAttribute(rnn_bwd_dh2d_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)DH2D_SMEM));
  const dim3 grid_dh((unsigned)((H + DH_U - 1) / DH_U), (unsigned)nparts, (unsigned)((B + BC - 1) / BC));
  int64_t eb = ((int64_t)B * H + RT - 1) / RT;
  if (eb > ctx->sm_count * 8) eb = ctx->sm_count * 8;
  for (int64_t t = persist ? -1 : T - 1; t >= 0; --t) {
    float* g_t = gates + t * 4 * H;
    const float* c_prev = t == 0 ? c0 : cst + (t - 1) * H;
    // recurrent dh entering step t: dhT at the last step, the partials of the step after it otherwise
    const float* dh_rec = (t == T - 1) ? dhT : parts;
    lstm_bwd_gates_kernel<<<(unsigned)eb, RT, 0, stream>>>(g_t, T * 4 * H, cst + t * H, c_prev, ldrow,
                                                           t == 0 ? (int64_t)H : ldrow, dout + t * H, ldrow, dh_rec,
                                                           (t == T - 1) ? 1 : nparts, dc, H, B);
    FB_LAUNCH_CHECK();
    if (t > 0) {
      rnn_bwd_dh2d_kernel<<<grid_dh, RT, DH2D_SMEM, stream>>>(Wh, g_t, T * 4 * H, parts, H, R, B);
      FB_LAUNCH_CHECK();
    }
  }
  // bulk GEMMs over all T*B columns (dg = gates buffer, [rows][4H])
  fb_gemm_args a;
  a.Z = nullptr; a.bias_n = nullptr; a.bias_m = nullptr; a.act = FB_ACT_IDENTITY; a.accumulate = 0;
  // dWi memory [in][4H] = x^T dg
  a.A = x; a.lda = in_dim; a.a_mn_major = 1;
  a.B = gates; a.ldb = 4 * hidden; a.b_mn_major = 1;
  a.C = dWi; a.ldc = 4 * hidden; a.M = in_dim; a.N = 4 * hidden; a.K = rows;
  st = fb_gemm_dispatch(ctx, stream, a, FB_PREC_DEFAULT);
  if (st != FB_OK) return st;
  // dWh memory [H][4H] = hprev^T dg with hprev(b, t) = out(b, t-1) (h0 at t = 0); the shifted copy lives in
  // the cache's input-projection region, which the backward pass no longer needs.
  {
    float* hprev_all = gates + rows * 5 * H;
    int64_t sb = (rows * H + RT - 1) / RT;
    if (sb > (int64_t)ctx->sm_count * 16) sb = (int64_t)ctx->sm_count * 16;
    shift_prev_kernel<<<(unsigned)sb, RT, 0, stream>>>(out, h0, hprev_all, H, T, batch);
    FB_LAUNCH_CHECK();
    a.A = hprev_all; a.lda = hidden; a.a_mn_major = 1;
    a.B = gates; a.ldb = 4 * hidden; a.b_mn_major = 1;
    a.C = dWh; a.ldc = 4 * hidden; a.M = hidden; a.N = 4 * hidden; a.K = rows;
    st = fb_gemm_dispatch(ctx, stream, a, FB_PREC_DEFAULT);
    if (st != FB_OK) return st;
  }
  a.accumulate = 0;
  if (db) {
    st = colsum_rows(ctx, stream, gates, db, rows, 4 * hidden);
    if (st != FB_OK) return st;
  }
  if (dx) {
    // dx[rows][in] = dg[rows][4H] * Wi (memory [in][4H]) ^T
    a.A = gates; a.lda = 4 * hidden; a.a_mn_major = 0;
    a.B = Wi; a.ldb = 4 * hidden; a.b_mn_major = 0;
    a.C = dx; a.ldc = in_dim; a.M = rows; a.N = in_dim; a.K = 4 * hidden;
    st = fb_gemm_dispatch(ctx, stream, a, FB_PREC_DEFAULT);
  }
  return st;
}

FB_API int32_t fb_gru_fwd(fb_ctx* ctx, void* stream_, const float* Wi, const float* Wh, const float* b, const float* x,
                          const float* h0, float* out, float* hT, void* cache, int64_t in_dim, int64_t hidden,
                          int64_t seq_len, int64_t batch) {
  FB_CHECK_CTX(ctx);
  cudaStream_t stream = (cudaStream_t)stream_;
  int32_t st = check_dims("fb_gru_fwd", in_dim, hidden, seq_len, batch);
  if (st != FB_OK) return st;
  if (seq_len == 0 || batch == 0) return FB_OK;
  FB_REQUIRE(Wi && Wh && x && out, FB_ERR_INVALID_ARG, "fb_gru_fwd: NULL pointer");
  const int H = (int)hidden, B = (int)batch;
  const int64_t T = seq_len, rows = T * batch, ldrow = T * H;
  float *cch = nullptr, *gx;
  if (cache) {
    cch = (float*)cache;
    gx = cch + rows * 4 * H;
  } else {
    gx = (float*)fb_scratch(ctx, stream, (size_t)(rows * 3 * H) * sizeof(float));
    if (!gx) return FB_ERR_ALLOC;
  }
  fb_gemm_args a;
  a.A = x; a.lda = in_dim; a.a_mn_major = 0;
  a.B = Wi; a.ldb = 3 * hidden; a.b_mn_major = 1;
  a.C = gx; a.ldc = 3 * hidden; a.Z = nullptr; a.bias_n = b; a.bias_m = nullptr;
  a.M = rows; a.N = 3 * hidden; a.K = in_dim; a.act = FB_ACT_IDENTITY; a.accumulate = 0;
  st = fb_gemm_dispatch(ctx, stream, a, FB_PREC_DEFAULT);
  if (st != FB_OK) return st;
  const bool fast = (H % 4 == 0) && fb_aligned16(Wh) && fb_aligned16(out) && (!h0 || fb_aligned16(h0)) &&
                    fast_fwd_smem(3, H) <= ctx->smem_optin;
  const int hu = fast ? 4 : pick_hu(3, H, ctx->smem_optin, (size_t)BC * HS * 4);
  FB_REQUIRE(hu > 0, FB_ERR_UNSUPPORTED, "fb_gru_fwd: hidden size %d does not fit the step kernel's shared memory", H);
  const size_t smem = fast ? fast_fwd_smem(3, H) : fwd_smem(3, hu, H);
  auto kern = hu == 4 ? gru_fwd_step_kernel<4> : hu == 2 ? gru_fwd_step_kernel<2> : gru_fwd_step_kernel<1>;
  if (fast) FB_CUDA(cudaFuncSetAttribute(gru_fwd_fast_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  else FB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  const unsigned grid = (unsigned)((H + hu - 1) / hu);
  if (fast && T > 1 && H % TU == 0 && B % TB == 0 && tile_fwd_smem(3, H) <= ctx->smem_optin && persistent_allowed(stream)) {
    // register-tiled persistent kernel: (H / 16) x (B / 16) blocks, all resident, one cooperative launch
    const int64_t tgrid = (int64_t)(H / TU) * (B / TB);
    const size_t tsmem = tile_fwd_smem(3, H);
    int per_sm = 0;
    FB_CUDA(cudaFuncSetAttribute(rnn_fwd_tile_kernel<3>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)tsmem));
    FB_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, rnn_fwd_tile_kernel<3>, RT, tsmem));
    if ((int64_t)per_sm * ctx->sm_count >= tgrid && T * tgrid < 0x7fffffff && B / TB <= 32) {
      unsigned* counter = (unsigned*)(ctx->dev_error + 16);      // one counter per batch group (at most 32)
      FB_CUDA(cudaMemsetAsync(counter, 0, (size_t)(B / TB) * sizeof(unsigned), stream));
      int cached = 0, Hi = H, Bi = B, Ti = (int)T;
      int32_t* dev_err = ctx->dev_error;
      const float* c0 = nullptr;
      float *cst = nullptr, *cT = nullptr;
      void* args[] = {(void*)&Wh, (void*)&gx, (void*)&h0, (void*)&c0, (void*)&out, (void*)&cch, (void*)&cst, (void*)&cached,
                      (void*)&hT, (void*)&cT, (void*)&Hi, (void*)&Bi, (void*)&Ti, (void*)&counter, (void*)&dev_err};
      FB_CUDA(launch_persistent((const void*)rnn_fwd_tile_kernel<3>, dim3((unsigned)tgrid), dim3(RT), args, tsmem, stream));
      FB_LAUNCH_CHECK();
      return FB_OK;
    }
  }
  if (fast && T > 1 && T * (int64_t)grid < 0x7fffffff && persistent_allowed(stream)) {
    // one cooperative launch for the whole sequence when every block can be resident at once
    int per_sm = 0;
    FB_CUDA(cudaFuncSetAttribute(gru_fwd_persist_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    FB_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, gru_fwd_persist_kernel, RT, smem));
    if ((int64_t)per_sm * ctx->sm_count >= (int64_t)grid) {
      unsigned* counter = (unsigned*)(ctx->dev_error + 16);
      FB_CUDA(cudaMemsetAsync(counter, 0, sizeof(unsigned), stream));
      int Hi = H, Bi = B, Ti = (int)T;
      int32_t* dev_err = ctx->dev_error;
      void* args[] = {(void*)&Wh, (void*)&gx, (void*)&h0, (void*)&out, (void*)&cch, (void*)&hT, (void*)&Hi, (void*)&Bi, (void*)&Ti,
                      (void*)&counter, (void*)&dev_err};
      FB_CUDA(launch_persistent((const void*)gru_fwd_persist_kernel, dim3(grid), dim3(RT), args, smem, stream));
      FB_LAUNCH_CHECK();
      return FB_OK;
    }
  }
  for (int64_t t = 0; t < T; ++t) {
    const float* hprev = t == 0 ? h0 : out + (t - 1) * H;
    const int64_t ldh = t == 0 ? H : ldrow;
    float* c_t = cch ? cch + t * 4 * H : nullptr;
    float* hT_t = (t == T - 1) ? hT : nullptr;
    if (fast)
      gru_fwd_fast_kernel<<<grid, RT, smem, stream>>>(Wh, gx + t * 3 * H, T * 3 * H, hprev, ldh, out + t * H, ldrow, c_t, T * 4 * H,
                                                      hT_t, H, B);
    else
      kern<<<grid, RT, smem, stream>>>(Wh, gx + t * 3 * H, T * 3 * H, hprev, ldh, out + t * H, ldrow, c_t, T * 4 * H, hT_t, H, B);
    FB_LAUNCH_CHECK();
  }
  return FB_OK;
}

FB_API int32_t fb_gru_bwd(fb_ctx* ctx, void* stream_, const float* Wi, const float* Wh, const float* x,
                          const float* h0, const float* out, const void* cache, const float* dout, const float* dhT, float* dWi, float* dWh, float* db,
                          float* dx, int64_t in_dim, int64_t hidden, int64_t seq_len, int64_t batch) {
  FB_CHECK_CTX(ctx);
  cudaStream_t stream = (cudaStream_t)stream_;
  int32_t st = check_dims("fb_gru_bwd", in_dim, hidden, seq_len, batch);
  if (st != FB_OK) return st;
  FB_REQUIRE(seq_len >= 1 && batch >= 1, FB_ERR_SHAPE, "fb_gru_bwd: empty sequence or batch");
  FB_REQUIRE(Wi && Wh && x && out && cache && dout && dWi && dWh, FB_ERR_INVALID_ARG, "fb_gru_bwd: NULL pointer");
  const int H = (int)hidden, B = (int)batch;
  const int64_t T = seq_len, rows = T * batch, ldrow = T * H;
  const float* cch = (const float*)cache;          // [rows][4H]
  float* dgx = (float*)cache + rows * 4 * H;       // [rows][3H], over the input projection
  float* dgh = dgx + rows * 3 * H;                 // [rows][3H]
  const int R = 3 * H;
  // one cooperative launch for the whole reverse time loop when its grid can be resident at once
  const int UBp = (H + DH_U - 1) / DH_U, NPp = (R + PB_R - 1) / PB_R, BZp = (B + BC - 1) / BC;
  const int64_t pgrid = (int64_t)UBp * NPp * BZp;
  bool persist = T > 1 && (H % 32 == 0) && fb_aligned16(Wh) && fb_aligned16(cache) && pgrid >= 1 && pgrid <= 4096 &&
                 2 * T * pgrid < 0x7fffffff && persistent_allowed(stream);
  if (persist) {
    int per_sm = 0;
    FB_CUDA(cudaFuncSetAttribute(gru_bwd_persist_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)PB_SMEM));
    FB_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, gru_bwd_persist_kernel, RT, PB_SMEM));
    persist = (int64_t)per_sm * ctx->sm_count >= pgrid;
  }
  const int nparts = persist ? NPp : (R + DH_R - 1) / DH_R;
  float* ws = (float*)fb_scratch(ctx, stream, (size_t)((1 + nparts) * (int64_t)B * H) * sizeof(float));
  if (!ws) return FB_ERR_ALLOC;
  float* dh_direct = ws;                     // dh * z, the part of dh_{t-1} that bypasses Wh
  float* parts = ws + (int64_t)B * H;        // [nparts][B][H] partial sums of Wh' * dgh
  if (persist) {
    unsigned* counter = (unsigned*)(ctx->dev_error + 16);
    FB_CUDA(cudaMemsetAsync(counter, 0, sizeof(unsigned), stream));
    int Hi = H, Bi = B, Ti = (int)T, ubi = UBp, npi = NPp;
    int32_t* dev_err = ctx->dev_error;
    void* args[] = {(void*)&Wh, (void*)&cch, (void*)&out, (void*)&h0, (void*)&dout, (void*)&dhT, (void*)&dgx, (void*)&dgh,
                    (void*)&dh_direct, (void*)&parts, (void*)&Hi, (void*)&Bi, (void*)&Ti, (void*)&ubi, (void*)&npi, (void*)&counter,
                    (void*)&dev_err};
    FB_CUDA(launch_persistent((const void*)gru_bwd_persist_kernel, dim3((unsigned)pgrid), dim3(RT), args, PB_SMEM, stream));
    FB_LAUNCH_CHECK();
  }
  FB_CUDA(cudaFuncSetAttribute(rnn_bwd_dh2d_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)DH2D_SMEM));
  const dim3 grid_dh((unsigned)((H + DH_U - 1) / DH_U), (unsigned)nparts, (unsigned)((B + BC - 1) / BC));
  int64_t eb = ((int64_t)B * H + RT - 1) / RT;
  if (eb > ctx->sm_count * 8) eb = ctx->sm_count * 8;
  for (int64_t t = persist ? -1 : T - 1; t >= 0; --t) {
    const float* hprev = t == 0 ? h0 : out + (t - 1) * H;
    const bool last = (t == T - 1);
    gru_bwd_gates_kernel<<<(unsigned)eb, RT, 0, stream>>>(cch + t * 4 * H, T * 4 * H, hprev, t == 0 ? (int64_t)H : ldrow,
                                                          dout + t * H, ldrow, last ? dhT : parts, last ? 1 : nparts,
                                                          last ? nullptr : dh_direct, dgx + t * 3 * H, dgh + t * 3 * H,
                                                          T * 3 * H, dh_direct, H, B);
    FB_LAUNCH_CHECK();
    if (t > 0) {
      rnn_bwd_dh2d_kernel<<<grid_dh, RT, DH2D_SMEM, stream>>>(Wh, dgh + t * 3 * H, T * 3 * H, parts, H, R, B);
      FB_LAUNCH_CHECK();
    }
  }
  fb_gemm_args a;
  a.Z = nullptr; a.bias_n = nullptr; a.bias_m = nullptr; a.act = FB_ACT_IDENTITY; a.accumulate = 0;
  a.A = x; a.lda = in_dim; a.a_mn_major = 1;
  a.B = dgx; a.ldb = 3 * hidden; a.b_mn_major = 1;
  a.C = dWi; a.ldc = 3 * hidden; a.M = in_dim; a.N = 3 * hidden; a.K = rows;
  st = fb_gemm_dispatch(ctx, stream, a, FB_PREC_DEFAULT);
  if (st != FB_OK) return st;
  {
    float* hprev_all = dgh + rows * 3 * H;
    int64_t sb = (rows * H + RT - 1) / RT;
    if (sb > (int64_t)ctx->sm_count * 16) sb = (int64_t)ctx->sm_count * 16;
    shift_prev_kernel<<<(unsigned)sb, RT, 0, stream>>>(out, h0, hprev_all, H, T, batch);
    FB_LAUNCH_CHECK();
    a.A = hprev_all; a.lda = hidden; a.a_mn_major = 1;
    a.B = dgh; a.ldb = 3 * hidden; a.b_mn_major = 1;
    a.C = dWh; a.ldc = 3 * hidden; a.M = hidden; a.N = 3 * hidden; a.K = rows;
    st = fb_gemm_dispatch(ctx, stream, a, FB_PREC_DEFAULT);
    if (st != FB_OK) return st;
  }
  a.accumulate = 0;
  if (db) {
    st = colsum_rows(ctx, stream, dgx, db, rows, 3 * hidden);
    if (st != FB_OK) return st;
  }
  if (dx) {
    a.A = dgx; a.lda = 3 * hidden; a.a_mn_major = 0;
    a.B = Wi; a.ldb = 3 * hidden; a.b_mn_major = 0;
    a.C = dx; a.ldc = in_dim; a.M = rows; a.N = in_dim; a.K = 3 * hidden;
    st = fb_gemm_dispatch(ctx, stream, a, FB_PREC_DEFAULT);
  }
  return st;
}
