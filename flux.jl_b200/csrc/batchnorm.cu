// BatchNorm forward (training / inference) and backward (memory-bound).
//
// Data layout: x is [n][c][s] row-major (Julia WHCN with s = W*H; a 2-D input [C, N] has s == 1).
// Training forward = statistics pass (read x) + finaliser (tiny) + normalise pass (read x, write y):
// 2 reads + 1 write.  Backward = reduction pass (read x, dy) + finaliser + dx pass (read x, dy, write
// dx): 4 reads + 1 write; the activation mask is recomputed from x instead of reading y.
// Statistics use a shifted sum / sum-of-squares per thread, converted to (count, mean, M2) and merged
// with Chan's (Welford) update through warp shuffles, so large |mean|/std inputs stay accurate.
#include "common.cuh"

namespace {

constexpr int BN_THREADS = 256;

struct Wf { float n, mean, m2; };

__device__ __forceinline__ Wf wf_warp_merge(Wf a) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float nb = __shfl_xor_sync(0xffffffffu, a.n, o);
    const float mb = __shfl_xor_sync(0xffffffffu, a.mean, o);
    const float qb = __shfl_xor_sync(0xffffffffu, a.m2, o);
    fb_welford_merge(a.n, a.mean, a.m2, nb, mb, qb);
  }
  return a;
}

// Block merge; result valid in thread 0.
__device__ __forceinline__ Wf wf_block_merge(Wf a, float* sh /* 96 floats */) {
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = blockDim.x >> 5;
  a = wf_warp_merge(a);
  __syncthreads();
  if (lane == 0) { sh[w] = a.n; sh[32 + w] = a.mean; sh[64 + w] = a.m2; }
  __syncthreads();
  Wf r;
  r.n = (lane < nw) ? sh[lane] : 0.0f;
  r.mean = (lane < nw) ? sh[32 + lane] : 0.0f;
  r.m2 = (lane < nw) ? sh[64 + lane] : 0.0f;
  return wf_warp_merge(r);
}

// --------------------------------------------------------------------------- statistics pass ---
// grid (c, split): block (ch, p) covers samples p, p+split, ... of channel ch.
template <bool VEC>
__global__ void __launch_bounds__(BN_THREADS)
bn_stats_kernel(const float* __restrict__ x, float* __restrict__ part /* [c][split][3] */, int64_t s,
                int64_t c, int64_t n) {
  __shared__ float sh[96];
  const int64_t ch = blockIdx.x;
  const int split = gridDim.y, p = blockIdx.y;
  const float shift = __ldg(x + ch * s);  // a value inside the channel's range
  float cnt = 0.0f, s1 = 0.0f, s2 = 0.0f;
  if (VEC) {
    // four rows per pass: four independent 128-bit loads in flight per thread
    const int64_t s4 = s >> 2;
    for (int64_t i = p; i < n; i += 4 * (int64_t)split) {
      const float4* r4[4];
      bool ok[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int64_t ii = i + (int64_t)u * split;
        ok[u] = ii < n;
        r4[u] = (const float4*)(x + ((ok[u] ? ii : i) * c + ch) * s);
      }
      for (int64_t j = threadIdx.x; j < s4; j += BN_THREADS) {
        float4 v[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) v[u] = ok[u] ? __ldcs(r4[u] + j) : make_float4(shift, shift, shift, shift);
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const float a = v[u].x - shift, b = v[u].y - shift, cc = v[u].z - shift, d = v[u].w - shift;
          s1 += (a + b) + (cc + d);
          s2 += (a * a + b * b) + (cc * cc + d * d);
          cnt += ok[u] ? 4.0f : 0.0f;
        }
      }
    }
  } else {
    for (int64_t i = p; i < n; i += split) {
      const float* row = x + (i * c + ch) * s;
      for (int64_t j = threadIdx.x; j < s; j += BN_THREADS) {
        const float a = row[j] - shift;
        s1 += a;
        s2 += a * a;
        cnt += 1.0f;
      }
    }
  }
  Wf w;
  w.n = cnt;
  w.mean = cnt > 0.0f ? s1 / cnt : 0.0f;
  w.m2 = cnt > 0.0f ? fmaxf(s2 - s1 * w.mean, 0.0f) : 0.0f;
  w.mean += shift;
  w = wf_block_merge(w, sh);
  if (threadIdx.x == 0) {
    float* o = part + (ch * split + p) * 3;
    o[0] = w.n; o[1] = w.mean; o[2] = w.m2;
  }
}

// One thread per channel: merge the split partials, write mean / rstd, update running statistics.
__global__ void bn_stats_finalize_kernel(const float* __restrict__ part, int split, int64_t c, float eps,
                                         float momentum, float* __restrict__ save_mean,
                                         float* __restrict__ save_rstd, float* __restrict__ running_mean,
                                         float* __restrict__ running_var) {
  const int64_t ch = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (ch >= c) return;
  float n = 0.0f, mean = 0.0f, m2 = 0.0f;
  for (int p = 0; p < split; ++p) {
    const float* q = part + (ch * split + p) * 3;
    fb_welford_merge(n, mean, m2, q[0], q[1], q[2]);
  }
  const float var = m2 / n;  // biased
  save_mean[ch] = mean;
  save_rstd[ch] = rsqrtf(var + eps);
  if (running_mean != nullptr) {
    running_mean[ch] = (1.0f - momentum) * running_mean[ch] + momentum * mean;
    running_var[ch] = (1.0f - momentum) * running_var[ch] + momentum * var * (n / (n - 1.0f));
  }
}

// rstd from running variance (inference)
__global__ void bn_infer_prepare_kernel(const float* __restrict__ running_mean, const float* __restrict__ running_var,
                                        float eps, int64_t c, float* __restrict__ mean, float* __restrict__ rstd) {
  const int64_t ch = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (ch >= c) return;
  mean[ch] = running_mean[ch];
  rstd[ch] = 1.0f / sqrtf(running_var[ch] + eps);
}

// ----------------------------------------------------------------------------- normalise pass ---
template <bool VEC>
__global__ void __launch_bounds__(BN_THREADS)
bn_apply_kernel(const float* __restrict__ x, const float* __restrict__ gamma, const float* __restrict__ beta,
                const float* __restrict__ mean, const float* __restrict__ rstd, float* __restrict__ y, int64_t s,
                int64_t c, int64_t total, int act) {
  if (VEC) {
    const int64_t total4 = total >> 2;
    const float4* x4 = (const float4*)x;
    float4* y4 = (float4*)y;
    for (int64_t i = (int64_t)blockIdx.x * BN_THREADS + threadIdx.x; i < total4; i += (int64_t)gridDim.x * BN_THREADS) {
      const int64_t ch = ((i << 2) / s) % c;
      const float mu = __ldg(mean + ch);
      const float sc = __ldg(rstd + ch) * (gamma ? __ldg(gamma + ch) : 1.0f);
      const float sf = beta ? __ldg(beta + ch) : 0.0f;
      const float4 v = __ldcs(x4 + i);
      float4 o;
      o.x = fmaf(v.x - mu, sc, sf); o.y = fmaf(v.y - mu, sc, sf); o.z = fmaf(v.z - mu, sc, sf); o.w = fmaf(v.w - mu, sc, sf);
      if (act != FB_ACT_IDENTITY) {
        o.x = fb_act_apply(act, o.x); o.y = fb_act_apply(act, o.y); o.z = fb_act_apply(act, o.z); o.w = fb_act_apply(act, o.w);
      }
      __stcs(y4 + i, o);
    }
  } else {
    for (int64_t i = (int64_t)blockIdx.x * BN_THREADS + threadIdx.x; i < total; i += (int64_t)gridDim.x * BN_THREADS) {
      const int64_t ch = (i / s) % c;
      const float sc = rstd[ch] * (gamma ? gamma[ch] : 1.0f);
      const float o = fmaf(x[i] - mean[ch], sc, beta ? beta[ch] : 0.0f);
      y[i] = fb_act_apply(act, o);
    }
  }
}

// Row-structured variants for long contiguous rows (s4 >= 32 float4): one (sample, channel) row per block pass, so
// the per-element channel lookup (an integer division) disappears; two rows per pass for memory-level parallelism.
__global__ void __launch_bounds__(BN_THREADS)
bn_apply_rows_kernel(const float4* __restrict__ x, const float* __restrict__ gamma, const float* __restrict__ beta,
                     const float* __restrict__ mean, const float* __restrict__ rstd, float4* __restrict__ y, int64_t s4,
                     int64_t c, int64_t rows, int act) {
  for (int64_t r0 = (int64_t)blockIdx.x * 2; r0 < rows; r0 += (int64_t)gridDim.x * 2) {
    const bool ok2 = r0 + 1 < rows;
    const int64_t ch0 = r0 % c, ch1 = (r0 + 1) % c;
    const float mu0 = __ldg(mean + ch0), sc0 = __ldg(rstd + ch0) * (gamma ? __ldg(gamma + ch0) : 1.0f), sf0 = beta ? __ldg(beta + ch0) : 0.0f;
    const float mu1 = __ldg(mean + ch1), sc1 = __ldg(rstd + ch1) * (gamma ? __ldg(gamma + ch1) : 1.0f), sf1 = beta ? __ldg(beta + ch1) : 0.0f;
    const float4* xa = x + r0 * s4;
    float4* ya = y + r0 * s4;
    for (int64_t j = threadIdx.x; j < s4; j += BN_THREADS) {
      const float4 va = __ldcs(xa + j);
      float4 vb = make_float4(0.f, 0.f, 0.f, 0.f);
      if (ok2) vb = __ldcs(xa + s4 + j);
      float4 oa, ob;
      oa.x = fmaf(va.x - mu0, sc0, sf0); oa.y = fmaf(va.y - mu0, sc0, sf0); oa.z = fmaf(va.z - mu0, sc0, sf0); oa.w = fmaf(va.w - mu0, sc0, sf0);
      ob.x = fmaf(vb.x - mu1, sc1, sf1); ob.y = fmaf(vb.y - mu1, sc1, sf1); ob.z = fmaf(vb.z - mu1, sc1, sf1); ob.w = fmaf(vb.w - mu1, sc1, sf1);
      if (act != FB_ACT_IDENTITY) {
        oa.x = fb_act_apply(act, oa.x); oa.y = fb_act_apply(act, oa.y); oa.z = fb_act_apply(act, oa.z); oa.w = fb_act_apply(act, oa.w);
        ob.x = fb_act_apply(act, ob.x); ob.y = fb_act_apply(act, ob.y); ob.z = fb_act_apply(act, ob.z); ob.w = fb_act_apply(act, ob.w);
      }
      __stcs(ya + j, oa);
      if (ok2) __stcs(ya + s4 + j, ob);
    }
  }
}

__global__ void __launch_bounds__(BN_THREADS)
bn_bwd_apply_rows_kernel(const float4* __restrict__ x, const float4* __restrict__ dy, const float* __restrict__ gamma,
                         const float* __restrict__ beta, const float* __restrict__ mean, const float* __restrict__ rstd,
                         const float* __restrict__ coef, float4* __restrict__ dx, int64_t s4, int64_t c, int64_t rows, int act) {
  for (int64_t r = blockIdx.x; r < rows; r += gridDim.x) {
    const int64_t ch = r % c;
    const float mu = __ldg(mean + ch), rs = __ldg(rstd + ch);
    const float ga = gamma ? __ldg(gamma + ch) : 1.0f, be = beta ? __ldg(beta + ch) : 0.0f;
    const float m1 = __ldg(coef + ch * 2), m2 = __ldg(coef + ch * 2 + 1), k = ga * rs;
    const float4* xa = x + r * s4;
    const float4* da = dy + r * s4;
    float4* oa = dx + r * s4;
    for (int64_t j = threadIdx.x; j < s4; j += 2 * BN_THREADS) {
      const int64_t j2 = j + BN_THREADS;
      const bool ok2 = j2 < s4;
      float4 xv[2], dz[2];
      xv[0] = __ldcs(xa + j); dz[0] = __ldcs(da + j);
      if (ok2) { xv[1] = __ldcs(xa + j2); dz[1] = __ldcs(da + j2); }
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        if (u == 1 && !ok2) break;
        const float h0 = (xv[u].x - mu) * rs, h1 = (xv[u].y - mu) * rs, h2 = (xv[u].z - mu) * rs, h3 = (xv[u].w - mu) * rs;
        if (act != FB_ACT_IDENTITY) {
          dz[u].x *= fb_act_grad_z(act, fmaf(h0, ga, be)); dz[u].y *= fb_act_grad_z(act, fmaf(h1, ga, be));
          dz[u].z *= fb_act_grad_z(act, fmaf(h2, ga, be)); dz[u].w *= fb_act_grad_z(act, fmaf(h3, ga, be));
        }
        float4 o;
        o.x = k * (dz[u].x - m1 - h0 * m2); o.y = k * (dz[u].y - m1 - h1 * m2);
        o.z = k * (dz[u].z - m1 - h2 * m2); o.w = k * (dz[u].w - m1 - h3 * m2);
        __stcs(oa + (u == 0 ? j : j2), o);
      }
    }
  }
}

// --------------------------------------------------------------------------- backward reduce ---
// part[c][split][2] = (sum dz, sum dz*xhat) with dz = dy * act'(gamma*xhat+beta)
template <bool VEC>
__global__ void __launch_bounds__(BN_THREADS)
bn_bwd_reduce_kernel(const float* __restrict__ x, const float* __restrict__ dy, const float* __restrict__ gamma,
                     const float* __restrict__ beta, const float* __restrict__ mean, const float* __restrict__ rstd,
                     float* __restrict__ part, int64_t s, int64_t c, int64_t n, int act) {
  __shared__ float sh[64];
  const int64_t ch = blockIdx.x;
  const int split = gridDim.y, p = blockIdx.y;
  const float mu = mean[ch], rs = rstd[ch];
  const float ga = gamma ? gamma[ch] : 1.0f, be = beta ? beta[ch] : 0.0f;
  float a1 = 0.0f, a2 = 0.0f;
  if (VEC) {
    const int64_t s4 = s >> 2;
    for (int64_t i = p; i < n; i += 2 * (int64_t)split) {
      const int64_t i2 = i + split;
      const bool ok2 = i2 < n;
      const float4* xa = (const float4*)(x + (i * c + ch) * s);
      const float4* da = (const float4*)(dy + (i * c + ch) * s);
      const float4* xb = (const float4*)(x + ((ok2 ? i2 : i) * c + ch) * s);
      const float4* db = (const float4*)(dy + ((ok2 ? i2 : i) * c + ch) * s);
      for (int64_t j = threadIdx.x; j < s4; j += BN_THREADS) {
        float4 xv[2], dz[2];
        xv[0] = __ldcs(xa + j); dz[0] = __ldcs(da + j);
        if (ok2) { xv[1] = __ldcs(xb + j); dz[1] = __ldcs(db + j); }
        else { xv[1] = make_float4(mu, mu, mu, mu); dz[1] = make_float4(0.f, 0.f, 0.f, 0.f); }
#pragma unroll
        for (int u = 0; u < 2; ++u) {
          const float h0 = (xv[u].x - mu) * rs, h1 = (xv[u].y - mu) * rs, h2 = (xv[u].z - mu) * rs, h3 = (xv[u].w - mu) * rs;
          if (act != FB_ACT_IDENTITY) {
            dz[u].x *= fb_act_grad_z(act, fmaf(h0, ga, be)); dz[u].y *= fb_act_grad_z(act, fmaf(h1, ga, be));
            dz[u].z *= fb_act_grad_z(act, fmaf(h2, ga, be)); dz[u].w *= fb_act_grad_z(act, fmaf(h3, ga, be));
          }
          a1 += (dz[u].x + dz[u].y) + (dz[u].z + dz[u].w);
          a2 += (dz[u].x * h0 + dz[u].y * h1) + (dz[u].z * h2 + dz[u].w * h3);
        }
      }
    }
  } else {
    for (int64_t i = p; i < n; i += split) {
      const int64_t base = (i * c + ch) * s;
      for (int64_t j = threadIdx.x; j < s; j += BN_THREADS) {
        const float h = (x[base + j] - mu) * rs;
        const float dz = dy[base + j] * fb_act_grad_z(act, fmaf(h, ga, be));
        a1 += dz;
        a2 += dz * h;
      }
    }
  }
  a1 = fb_warp_sum(a1);
  a2 = fb_warp_sum(a2);
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  if (lane == 0) { sh[w] = a1; sh[32 + w] = a2; }
  __syncthreads();
  if (w == 0) {
    float r1 = lane < (BN_THREADS / 32) ? sh[lane] : 0.0f;
    float r2 = lane < (BN_THREADS / 32) ? sh[32 + lane] : 0.0f;
    r1 = fb_warp_sum(r1);
    r2 = fb_warp_sum(r2);
    if (lane == 0) {
      part[(ch * split + p) * 2 + 0] = r1;
      part[(ch * split + p) * 2 + 1] = r2;
    }
  }
}

// coef[c][2] = (sum dz / cnt, sum dz*xhat / cnt); dgamma, dbeta
__global__ void bn_bwd_finalize_kernel(const float* __restrict__ part, int split, int64_t c, float cnt,
                                       float* __restrict__ coef, float* __restrict__ dgamma,
                                       float* __restrict__ dbeta) {
  const int64_t ch = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (ch >= c) return;
  float a1 = 0.0f, a2 = 0.0f;
  for (int p = 0; p < split; ++p) {
    a1 += part[(ch * split + p) * 2 + 0];
    a2 += part[(ch * split + p) * 2 + 1];
  }
  if (dbeta) dbeta[ch] = a1;
  if (dgamma) dgamma[ch] = a2;
  coef[ch * 2 + 0] = a1 / cnt;
  coef[ch * 2 + 1] = a2 / cnt;
}

template <bool VEC>
__global__ void __launch_bounds__(BN_THREADS)
bn_bwd_apply_kernel(const float* __restrict__ x, const float* __restrict__ dy, const float* __restrict__ gamma,
                    const float* __restrict__ beta, const float* __restrict__ mean, const float* __restrict__ rstd,
                    const float* __restrict__ coef, float* __restrict__ dx, int64_t s, int64_t c, int64_t total,
                    int act) {
  if (VEC) {
    const int64_t total4 = total >> 2;
    const float4* x4 = (const float4*)x;
    const float4* d4 = (const float4*)dy;
    float4* o4 = (float4*)dx;
    for (int64_t i = (int64_t)blockIdx.x * BN_THREADS + threadIdx.x; i < total4; i += (int64_t)gridDim.x * BN_THREADS) {
      const int64_t ch = ((i << 2) / s) % c;
      const float mu = __ldg(mean + ch), rs = __ldg(rstd + ch);
      const float ga = gamma ? __ldg(gamma + ch) : 1.0f, be = beta ? __ldg(beta + ch) : 0.0f;
      const float m1 = __ldg(coef + ch * 2), m2 = __ldg(coef + ch * 2 + 1);
      const float4 xv = __ldcs(x4 + i);
      float4 dz = __ldcs(d4 + i);
      const float h0 = (xv.x - mu) * rs, h1 = (xv.y - mu) * rs, h2 = (xv.z - mu) * rs, h3 = (xv.w - mu) * rs;
      if (act != FB_ACT_IDENTITY) {
        dz.x *= fb_act_grad_z(act, fmaf(h0, ga, be)); dz.y *= fb_act_grad_z(act, fmaf(h1, ga, be));
        dz.z *= fb_act_grad_z(act, fmaf(h2, ga, be)); dz.w *= fb_act_grad_z(act, fmaf(h3, ga, be));
      }
      const float k = ga * rs;
      float4 o;
      o.x = k * (dz.x - m1 - h0 * m2); o.y = k * (dz.y - m1 - h1 * m2);
      o.z = k * (dz.z - m1 - h2 * m2); o.w = k * (dz.w - m1 - h3 * m2);
      __stcs(o4 + i, o);
    }
  } else {
    for (int64_t i = (int64_t)blockIdx.x * BN_THREADS + threadIdx.x; i < total; i += (int64_t)gridDim.x * BN_THREADS) {
      const int64_t ch = (i / s) % c;
      const float rs = rstd[ch], ga = gamma ? gamma[ch] : 1.0f, be = beta ? beta[ch] : 0.0f;
      const float h = (x[i] - mean[ch]) * rs;
      const float dz = dy[i] * fb_act_grad_z(act, fmaf(h, ga, be));
      dx[i] = ga * rs * (dz - coef[ch * 2] - h * coef[ch * 2 + 1]);
    }
  }
}

int bn_pick_split(const fb_ctx* ctx, int64_t c, int64_t n) {
  int64_t target = (int64_t)ctx->sm_count * 8;
  int64_t split = (target + c - 1) / c;
  if (split < 1) split = 1;
  if (split > n) split = n;
  if (split > 65535) split = 65535;
  return (int)split;
}

unsigned bn_elem_grid(const fb_ctx* ctx, int64_t work_items) {
  int64_t blocks = (work_items + BN_THREADS - 1) / BN_THREADS;
  const int64_t cap = (int64_t)ctx->sm_count * 32;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  return (unsigned)blocks;
}

unsigned bn_row_grid(const fb_ctx* ctx, int64_t rows) {
  int64_t blocks = (rows + 1) / 2;
  const int64_t cap = (int64_t)ctx->sm_count * 16;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  return (unsigned)blocks;
}

int32_t bn_check(const char* fn, int64_t s, int64_t c, int64_t n, int act) {
  FB_REQUIRE(s >= 1 && c >= 1 && n >= 0, FB_ERR_SHAPE, "%s: bad shape s=%lld c=%lld n=%lld", fn, (long long)s,
             (long long)c, (long long)n);
  FB_REQUIRE(c <= 0x7fffffff, FB_ERR_SHAPE, "%s: too many channels", fn);
  FB_REQUIRE(fb_act_valid(act), FB_ERR_INVALID_ARG, "%s: unknown activation %d", fn, act);
  return FB_OK;
}

}  // namespace

FB_API int32_t fb_batchnorm_fwd_train(fb_ctx* ctx, void* stream_, const float* x, const float* gamma,
                                      const float* beta, float* running_mean, float* running_var, float* y,
                                      float* save_mean, float* save_rstd, int64_t s, int64_t c, int64_t n,
                                      float eps, float momentum, int32_t act, int32_t track_stats) {
  FB_CHECK_CTX(ctx);
  cudaStream_t stream = (cudaStream_t)stream_;
  int32_t st = bn_check("fb_batchnorm_fwd_train", s, c, n, act);
  if (st != FB_OK) return st;
  FB_REQUIRE((gamma == nullptr) == (beta == nullptr), FB_ERR_INVALID_ARG, "fb_batchnorm_fwd_train: gamma and beta must both be given or both NULL");
  FB_REQUIRE(s * n > 1, FB_ERR_SHAPE,
             "fb_batchnorm_fwd_train: BatchNorm expected more than 1 value per channel when training, got s*n = %lld",
             (long long)(s * n));
  FB_REQUIRE(x && y && save_mean && save_rstd, FB_ERR_INVALID_ARG, "fb_batchnorm_fwd_train: NULL pointer");
  FB_REQUIRE((running_mean == nullptr) == (running_var == nullptr), FB_ERR_INVALID_ARG, "fb_batchnorm_fwd_train: running_mean and running_var must both be given or both NULL");
  const int split = bn_pick_split(ctx, c, n);
  float* part = (float*)fb_scratch(ctx, stream, (size_t)c * split * 3 * sizeof(float));
  if (!part) return FB_ERR_ALLOC;
  const bool vec = (s % 4 == 0) && fb_aligned16(x) && fb_aligned16(y);
  dim3 grid((unsigned)c, (unsigned)split);
  if (vec) bn_stats_kernel<true><<<grid, BN_THREADS, 0, stream>>>(x, part, s, c, n);
  else bn_stats_kernel<false><<<grid, BN_THREADS, 0, stream>>>(x, part, s, c, n);
  FB_LAUNCH_CHECK();
  const bool upd = track_stats != 0 && running_mean != nullptr;
  bn_stats_finalize_kernel<<<(unsigned)((c + 127) / 128), 128, 0, stream>>>(part, split, c, eps, momentum, save_mean,
                                                                           save_rstd, upd ? running_mean : nullptr,
                                                                           upd ? running_var : nullptr);
  FB_LAUNCH_CHECK();
  const int64_t total = s * c * n;
  if (vec && s >= 128) bn_apply_rows_kernel<<<bn_row_grid(ctx, c * n), BN_THREADS, 0, stream>>>((const float4*)x, gamma, beta, save_mean, save_rstd, (float4*)y, s / 4, c, c * n, act);
  else if (vec) bn_apply_kernel<true><<<bn_elem_grid(ctx, total / 4), BN_THREADS, 0, stream>>>(x, gamma, beta, save_mean, save_rstd, y, s, c, total, act);
  else bn_apply_kernel<false><<<bn_elem_grid(ctx, total), BN_THREADS, 0, stream>>>(x, gamma, beta, save_mean, save_rstd, y, s, c, total, act);
  FB_LAUNCH_CHECK();
  return FB_OK;
}

FB_API int32_t fb_batchnorm_fwd_infer(fb_ctx* ctx, void* stream_, const float* x, const float* gamma,
                                      const float* beta, const float* running_mean, const float* running_var,
                                      float* y, int64_t s, int64_t c, int64_t n, float eps, int32_t act) {
  FB_CHECK_CTX(ctx);
  cudaStream_t stream = (cudaStream_t)stream_;
  int32_t st = bn_check("fb_batchnorm_fwd_infer", s, c, n, act);
  if (st != FB_OK) return st;
  FB_REQUIRE((gamma == nullptr) == (beta == nullptr), FB_ERR_INVALID_ARG, "fb_batchnorm_fwd_infer: gamma and beta must both be given or both NULL");
  if (n == 0) return FB_OK;
  FB_REQUIRE(x && y, FB_ERR_INVALID_ARG, "fb_batchnorm_fwd_infer: NULL pointer");
  const int split = bn_pick_split(ctx, c, n);
  float* ws = (float*)fb_scratch(ctx, stream, (size_t)c * (split * 3 + 2) * sizeof(float));
  if (!ws) return FB_ERR_ALLOC;
  float* mean = ws;
  float* rstd = ws + c;
  float* part = ws + 2 * c;
  const bool vec = (s % 4 == 0) && fb_aligned16(x) && fb_aligned16(y);
  if (running_mean != nullptr && running_var != nullptr) {
    bn_infer_prepare_kernel<<<(unsigned)((c + 127) / 128), 128, 0, stream>>>(running_mean, running_var, eps, c, mean, rstd);
  } else {
    dim3 grid((unsigned)c, (unsigned)split);
    if (vec) bn_stats_kernel<true><<<grid, BN_THREADS, 0, stream>>>(x, part, s, c, n);
    else bn_stats_kernel<false><<<grid, BN_THREADS, 0, stream>>>(x, part, s, c, n);
    FB_LAUNCH_CHECK();
    bn_stats_finalize_kernel<<<(unsigned)((c + 127) / 128), 128, 0, stream>>>(part, split, c, eps, 0.0f, mean, rstd, nullptr, nullptr);
  }
  FB_LAUNCH_CHECK();
  const int64_t total = s * c * n;
  if (vec && s >= 128) bn_apply_rows_kernel<<<bn_row_grid(ctx, c * n), BN_THREADS, 0, stream>>>((const float4*)x, gamma, beta, mean, rstd, (float4*)y, s / 4, c, c * n, act);
  else if (vec) bn_apply_kernel<true><<<bn_elem_grid(ctx, total / 4), BN_THREADS, 0, stream>>>(x, gamma, beta, mean, rstd, y, s, c, total, act);
  else bn_apply_kernel<false><<<bn_elem_grid(ctx, total), BN_THREADS, 0, stream>>>(x, gamma, beta, mean, rstd, y, s, c, total, act);
  FB_LAUNCH_CHECK();
  return FB_OK;
}

FB_API int32_t fb_batchnorm_bwd(fb_ctx* ctx, void* stream_, const float* x, const float* gamma,
                                const float* beta, const float* save_mean, const float* save_rstd,
                                const float* dy, float* dx, float* dgamma, float* dbeta, int64_t s, int64_t c,
                                int64_t n, int32_t act) {
  FB_CHECK_CTX(ctx);
  cudaStream_t stream = (cudaStream_t)stream_;
  int32_t st = bn_check("fb_batchnorm_bwd", s, c, n, act);
  if (st != FB_OK) return st;
  FB_REQUIRE((gamma == nullptr) == (beta == nullptr), FB_ERR_INVALID_ARG, "fb_batchnorm_bwd: gamma and beta must both be given or both NULL");
  FB_REQUIRE(n >= 1, FB_ERR_SHAPE, "fb_batchnorm_bwd: empty batch");
  FB_REQUIRE(x && save_mean && save_rstd && dy && dx, FB_ERR_INVALID_ARG, "fb_batchnorm_bwd: NULL pointer");
  const int split = bn_pick_split(ctx, c, n);
  float* ws = (float*)fb_scratch(ctx, stream, (size_t)c * (split * 2 + 2) * sizeof(float));
  if (!ws) return FB_ERR_ALLOC;
  float* coef = ws;
  float* part = ws + 2 * c;
  const bool vec = (s % 4 == 0) && fb_aligned16(x) && fb_aligned16(dy) && fb_aligned16(dx);
  dim3 grid((unsigned)c, (unsigned)split);
  if (vec) bn_bwd_reduce_kernel<true><<<grid, BN_THREADS, 0, stream>>>(x, dy, gamma, beta, save_mean, save_rstd, part, s, c, n, act);
  else bn_bwd_reduce_kernel<false><<<grid, BN_THREADS, 0, stream>>>(x, dy, gamma, beta, save_mean, save_rstd, part, s, c, n, act);
  FB_LAUNCH_CHECK();
  bn_bwd_finalize_kernel<<<(unsigned)((c + 127) / 128), 128, 0, stream>>>(part, split, c, (float)(s * n), coef, dgamma, dbeta);
  FB_LAUNCH_CHECK();
  const int64_t total = s * c * n;
  if (vec && s >= 128) bn_bwd_apply_rows_kernel<<<bn_row_grid(ctx, c * n), BN_THREADS, 0, stream>>>((const float4*)x, (const float4*)dy, gamma, beta, save_mean, save_rstd, coef, (float4*)dx, s / 4, c, c * n, act);
  else if (vec) bn_bwd_apply_kernel<true><<<bn_elem_grid(ctx, total / 4), BN_THREADS, 0, stream>>>(x, dy, gamma, beta, save_mean, save_rstd, coef, dx, s, c, total, act);
  else bn_bwd_apply_kernel<false><<<bn_elem_grid(ctx, total), BN_THREADS, 0, stream>>>(x, dy, gamma, beta, save_mean, save_rstd, coef, dx, s, c, total, act);
  FB_LAUNCH_CHECK();
  return FB_OK;
}
