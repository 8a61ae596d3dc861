// LayerNorm forward / backward (memory-bound).
//
// Data layout: x is [n][d] row-major (Julia x[d, n]); statistics run over the d contiguous floats of a
// row.  Forward: one read of x, one write of y (the row lives in registers between the two reductions).
// Backward: one read each of x and dy, one write of dx; dgamma / dbeta are accumulated per thread in
// registers across the rows a block owns and reduced in a second, small kernel from per-block partials.
#include "common.cuh"

namespace {

constexpr int LN_THREADS = 256;

__device__ __forceinline__ float4 ld_stream(const float4* p) { return __ldcs(p); }
__device__ __forceinline__ void st_stream(float4* p, float4 v) { __stcs(p, v); }

// Two block-wide sums at once.  sh must hold 64 floats.
__device__ __forceinline__ void block_sum2(float& a, float& b, float* sh) {
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = blockDim.x >> 5;
  a = fb_warp_sum(a);
  b = fb_warp_sum(b);
  __syncthreads();
  if (lane == 0) { sh[w] = a; sh[32 + w] = b; }
  __syncthreads();
  float ra = (lane < nw) ? sh[lane] : 0.0f;
  float rb = (lane < nw) ? sh[32 + lane] : 0.0f;
  a = fb_warp_sum(ra);
  b = fb_warp_sum(rb);
}

// ------------------------------------------------------------------ forward, row in registers ---
template <int V>
__global__ void __launch_bounds__(LN_THREADS)
ln_fwd_vec_kernel(const float4* __restrict__ x, const float4* __restrict__ gamma,
                  const float4* __restrict__ beta, float4* __restrict__ y, float* __restrict__ mean,
                  float* __restrict__ rstd, int d4, int64_t n, float eps, int act) {
  __shared__ float sh[64];
  const float inv_d = 1.0f / (4.0f * (float)d4);
  for (int64_t row = blockIdx.x; row < n; row += gridDim.x) {
    const float4* xr = x + row * d4;
    float4 v[V];
    float s = 0.0f;
#pragma unroll
    for (int i = 0; i < V; ++i) {
      const int c = threadIdx.x + i * LN_THREADS;
      if (c < d4) {
        v[i] = ld_stream(xr + c);
        s += (v[i].x + v[i].y) + (v[i].z + v[i].w);
      } else {
        v[i] = make_float4(0.f, 0.f, 0.f, 0.f);
      }
    }
    const float mu = fb_block_sum(s, sh) * inv_d;
    float q = 0.0f;
#pragma unroll
    for (int i = 0; i < V; ++i) {
      const int c = threadIdx.x + i * LN_THREADS;
      if (c < d4) {
        const float a = v[i].x - mu, b = v[i].y - mu, cc = v[i].z - mu, dd = v[i].w - mu;
        q += (a * a + b * b) + (cc * cc + dd * dd);
      }
    }
    const float var = fb_block_sum(q, sh) * inv_d;
    const float rs = rsqrtf(var + eps);
    if (threadIdx.x == 0) {
      mean[row] = mu;
      rstd[row] = rs;
    }
    float4* yr = y + row * d4;
#pragma unroll
    for (int i = 0; i < V; ++i) {
      const int c = threadIdx.x + i * LN_THREADS;
      if (c < d4) {
        float4 o;
        o.x = (v[i].x - mu) * rs; o.y = (v[i].y - mu) * rs; o.z = (v[i].z - mu) * rs; o.w = (v[i].w - mu) * rs;
        if (gamma != nullptr) {
          const float4 g = __ldg(gamma + c), b = __ldg(beta + c);
          o.x = fmaf(o.x, g.x, b.x); o.y = fmaf(o.y, g.y, b.y); o.z = fmaf(o.z, g.z, b.z); o.w = fmaf(o.w, g.w, b.w);
        }
        if (act != FB_ACT_IDENTITY) {
          o.x = fb_act_apply(act, o.x); o.y = fb_act_apply(act, o.y);
          o.z = fb_act_apply(act, o.z); o.w = fb_act_apply(act, o.w);
        }
        st_stream(yr + c, o);
      }
    }
  }
}

// ------------------------------------------------------------------ forward, any d / alignment ---
__global__ void __launch_bounds__(LN_THREADS)
ln_fwd_generic_kernel(const float* __restrict__ x, const float* __restrict__ gamma,
                      const float* __restrict__ beta, float* __restrict__ y, float* __restrict__ mean,
                      float* __restrict__ rstd, int64_t d, int64_t n, float eps, int act) {
  __shared__ float sh[64];
  for (int64_t row = blockIdx.x; row < n; row += gridDim.x) {
    const float* xr = x + row * d;
    float s = 0.0f;
    for (int64_t c = threadIdx.x; c < d; c += LN_THREADS) s += xr[c];
    const float mu = fb_block_sum(s, sh) / (float)d;
    float q = 0.0f;
    for (int64_t c = threadIdx.x; c < d; c += LN_THREADS) { const float a = xr[c] - mu; q += a * a; }
    const float var = fb_block_sum(q, sh) / (float)d;
    const float rs = rsqrtf(var + eps);
    if (threadIdx.x == 0) { mean[row] = mu; rstd[row] = rs; }
    float* yr = y + row * d;
    for (int64_t c = threadIdx.x; c < d; c += LN_THREADS) {
      float o = (xr[c] - mu) * rs;
      if (gamma != nullptr) o = fmaf(o, gamma[c], beta[c]);
      yr[c] = fb_act_apply(act, o);
    }
  }
}

// ----------------------------------------------------------------- backward, row in registers ---
template <int V>
__global__ void __launch_bounds__(LN_THREADS, 2)
ln_bwd_vec_kernel(const float4* __restrict__ x, const float4* __restrict__ gamma,
                  const float4* __restrict__ beta, const float* __restrict__ mean,
                  const float* __restrict__ rstd, const float4* __restrict__ dy, float4* __restrict__ dx,
                  float4* __restrict__ part_dg, float4* __restrict__ part_db, int d4, int64_t n, int act) {
  __shared__ float sh[64];
  const float inv_d = 1.0f / (4.0f * (float)d4);
  float4 ag[V], ab[V], gam[V], bet[V];
#pragma unroll
  for (int i = 0; i < V; ++i) {
    const int c = threadIdx.x + i * LN_THREADS;
    ag[i] = make_float4(0.f, 0.f, 0.f, 0.f);
    ab[i] = make_float4(0.f, 0.f, 0.f, 0.f);
    gam[i] = (gamma != nullptr && c < d4) ? __ldg(gamma + c) : make_float4(1.f, 1.f, 1.f, 1.f);
    bet[i] = (beta != nullptr && c < d4) ? __ldg(beta + c) : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  for (int64_t row = blockIdx.x; row < n; row += gridDim.x) {
    const float mu = __ldg(mean + row), rs = __ldg(rstd + row);
    const float4* xr = x + row * d4;
    const float4* dyr = dy + row * d4;
    float4 xh[V], g[V];
    float s1 = 0.0f, s2 = 0.0f;
#pragma unroll
    for (int i = 0; i < V; ++i) {
      const int c = threadIdx.x + i * LN_THREADS;
      if (c < d4) {
        const float4 xv = ld_stream(xr + c);
        float4 dz = ld_stream(dyr + c);
        xh[i].x = (xv.x - mu) * rs; xh[i].y = (xv.y - mu) * rs; xh[i].z = (xv.z - mu) * rs; xh[i].w = (xv.w - mu) * rs;
        if (act != FB_ACT_IDENTITY) {
          dz.x *= fb_act_grad_z(act, fmaf(xh[i].x, gam[i].x, bet[i].x));
          dz.y *= fb_act_grad_z(act, fmaf(xh[i].y, gam[i].y, bet[i].y));
          dz.z *= fb_act_grad_z(act, fmaf(xh[i].z, gam[i].z, bet[i].z));
          dz.w *= fb_act_grad_z(act, fmaf(xh[i].w, gam[i].w, bet[i].w));
        }
        ag[i].x = fmaf(dz.x, xh[i].x, ag[i].x); ag[i].y = fmaf(dz.y, xh[i].y, ag[i].y);
        ag[i].z = fmaf(dz.z, xh[i].z, ag[i].z); ag[i].w = fmaf(dz.w, xh[i].w, ag[i].w);
        ab[i].x += dz.x; ab[i].y += dz.y; ab[i].z += dz.z; ab[i].w += dz.w;
        g[i].x = dz.x * gam[i].x; g[i].y = dz.y * gam[i].y; g[i].z = dz.z * gam[i].z; g[i].w = dz.w * gam[i].w;
        s1 += (g[i].x + g[i].y) + (g[i].z + g[i].w);
        s2 += (g[i].x * xh[i].x + g[i].y * xh[i].y) + (g[i].z * xh[i].z + g[i].w * xh[i].w);
      }
    }
    block_sum2(s1, s2, sh);
    const float m1 = s1 * inv_d, m2 = s2 * inv_d;
    float4* dxr = dx + row * d4;
#pragma unroll
    for (int i = 0; i < V; ++i) {
      const int c = threadIdx.x + i * LN_THREADS;
      if (c < d4) {
        float4 o;
        o.x = rs * (g[i].x - m1 - xh[i].x * m2); o.y = rs * (g[i].y - m1 - xh[i].y * m2);
        o.z = rs * (g[i].z - m1 - xh[i].z * m2); o.w = rs * (g[i].w - m1 - xh[i].w * m2);
        st_stream(dxr + c, o);
      }
    }
  }
  if (part_dg != nullptr) {
#pragma unroll
    for (int i = 0; i < V; ++i) {
      const int c = threadIdx.x + i * LN_THREADS;
      if (c < d4) {
        part_dg[(int64_t)blockIdx.x * d4 + c] = ag[i];
        part_db[(int64_t)blockIdx.x * d4 + c] = ab[i];
      }
    }
  }
}

// ------------------------------------------- backward, rows staged through shared memory ---
// Same arithmetic as ln_bwd_vec_kernel, but the x and dy rows of the next LN_PIPE - 1 iterations are already in
// flight (cp.async.bulk into a ring of shared-memory stages) while the current row is reduced, so the kernel does
// not depend on occupancy for memory-level parallelism.
constexpr int LN_PIPE_MAX = 3;
constexpr uint32_t LN_WAIT_LIMIT = 1u << 22;

__device__ __forceinline__ uint32_t ln_smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

template <int V>
__global__ void __launch_bounds__(LN_THREADS, 2)
ln_bwd_pipe_kernel(const float* __restrict__ x, const float4* __restrict__ gamma, const float4* __restrict__ beta,
                   const float* __restrict__ mean, const float* __restrict__ rstd, const float* __restrict__ dy,
                   float4* __restrict__ dx, float4* __restrict__ part_dg, float4* __restrict__ part_db, int d4,
                   int64_t n, int act, int nstages, int32_t* __restrict__ dev_err) {
  extern __shared__ __align__(128) uint8_t ln_smem[];
  __shared__ float sh[64];
  __shared__ __align__(8) uint64_t bar[LN_PIPE_MAX];
  __shared__ int s_fail;
  const uint32_t row_bytes = (uint32_t)d4 * 16u;
  float4* stage_base = (float4*)ln_smem;                 // stage s: x row at [s][0], dy row at [s][1]
  const float inv_d = 1.0f / (4.0f * (float)d4);
  const int64_t first = blockIdx.x, step = gridDim.x;
  const int64_t my_rows = first < n ? (n - first + step - 1) / step : 0;

  auto issue = [&](int64_t i) {   // one thread: bring row first + i*step into stage i % nstages
    const int s = (int)(i % nstages);
    const int64_t row = first + i * step;
    const uint32_t b = ln_smem_u32(&bar[s]);
    const uint32_t dst_x = ln_smem_u32(stage_base + (size_t)(2 * s) * d4);
    const uint32_t dst_d = ln_smem_u32(stage_base + (size_t)(2 * s + 1) * d4);
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(b), "r"(2u * row_bytes) : "memory");
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst_x), "l"(x + row * (int64_t)d4 * 4), "r"(row_bytes), "r"(b) : "memory");
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst_d), "l"(dy + row * (int64_t)d4 * 4), "r"(row_bytes), "r"(b) : "memory");
  };

  if (threadIdx.x == 0) {
    for (int s = 0; s < nstages; ++s)
      asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(ln_smem_u32(&bar[s])) : "memory");
    s_fail = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    for (int64_t i = 0; i < nstages && i < my_rows; ++i) issue(i);
  }
  __syncthreads();

  float4 ag[V], ab[V], gam[V], bet[V];
#pragma unroll
  for (int i = 0; i < V; ++i) {
    const int c = threadIdx.x + i * LN_THREADS;
    ag[i] = make_float4(0.f, 0.f, 0.f, 0.f);
    ab[i] = make_float4(0.f, 0.f, 0.f, 0.f);
    gam[i] = (gamma != nullptr && c < d4) ? __ldg(gamma + c) : make_float4(1.f, 1.f, 1.f, 1.f);
    bet[i] = (beta != nullptr && c < d4) ? __ldg(beta + c) : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  for (int64_t it = 0; it < my_rows; ++it) {
    const int s = (int)(it % nstages);
    const uint32_t parity = (uint32_t)(it / nstages) & 1u;
    const int64_t row = first + it * step;
    {
      // bounded wait for this stage's two bulk copies
      const uint32_t b = ln_smem_u32(&bar[s]);
      uint32_t ok = 0;
      for (uint32_t spin = 0; spin < LN_WAIT_LIMIT && !ok; ++spin)
        asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                     : "=r"(ok) : "r"(b), "r"(parity) : "memory");
      if (!ok) s_fail = 1;
    }
    const float mu = __ldg(mean + row), rs = __ldg(rstd + row);
    const float4* xr = stage_base + (size_t)(2 * s) * d4;
    const float4* dyr = stage_base + (size_t)(2 * s + 1) * d4;
    float4 xh[V], g[V];
    float s1 = 0.0f, s2 = 0.0f;
#pragma unroll
    for (int i = 0; i < V; ++i) {
      const int c = threadIdx.x + i * LN_THREADS;
      if (c < d4) {
        const float4 xv = xr[c];
        float4 dz = dyr[c];
        xh[i].x = (xv.x - mu) * rs; xh[i].y = (xv.y - mu) * rs; xh[i].z = (xv.z - mu) * rs; xh[i].w = (xv.w - mu) * rs;
        if (act != FB_ACT_IDENTITY) {
          dz.x *= fb_act_grad_z(act, fmaf(xh[i].x, gam[i].x, bet[i].x));
          dz.y *= fb_act_grad_z(act, fmaf(xh[i].y, gam[i].y, bet[i].y));
          dz.z *= fb_act_grad_z(act, fmaf(xh[i].z, gam[i].z, bet[i].z));
          dz.w *= fb_act_grad_z(act, fmaf(xh[i].w, gam[i].w, bet[i].w));
        }
        ag[i].x = fmaf(dz.x, xh[i].x, ag[i].x); ag[i].y = fmaf(dz.y, xh[i].y, ag[i].y);
        ag[i].z = fmaf(dz.z, xh[i].z, ag[i].z); ag[i].w = fmaf(dz.w, xh[i].w, ag[i].w);
        ab[i].x += dz.x; ab[i].y += dz.y; ab[i].z += dz.z; ab[i].w += dz.w;
        g[i].x = dz.x * gam[i].x; g[i].y = dz.y * gam[i].y; g[i].z = dz.z * gam[i].z; g[i].w = dz.w * gam[i].w;
        s1 += (g[i].x + g[i].y) + (g[i].z + g[i].w);
        s2 += (g[i].x * xh[i].x + g[i].y * xh[i].y) + (g[i].z * xh[i].z + g[i].w * xh[i].w);
      }
    }
    block_sum2(s1, s2, sh);   // its barriers also mean: every thread has finished reading stage s
    if (s_fail) break;        // block-uniform after the barriers above
    if (threadIdx.x == 0 && it + nstages < my_rows) issue(it + nstages);
    const float m1 = s1 * inv_d, m2 = s2 * inv_d;
    float4* dxr = dx + row * d4;
#pragma unroll
    for (int i = 0; i < V; ++i) {
      const int c = threadIdx.x + i * LN_THREADS;
      if (c < d4) {
        float4 o;
        o.x = rs * (g[i].x - m1 - xh[i].x * m2); o.y = rs * (g[i].y - m1 - xh[i].y * m2);
        o.z = rs * (g[i].z - m1 - xh[i].z * m2); o.w = rs * (g[i].w - m1 - xh[i].w * m2);
        st_stream(dxr + c, o);
      }
    }
  }
  if (part_dg != nullptr) {
#pragma unroll
    for (int i = 0; i < V; ++i) {
      const int c = threadIdx.x + i * LN_THREADS;
      if (c < d4) {
        part_dg[(int64_t)blockIdx.x * d4 + c] = ag[i];
        part_db[(int64_t)blockIdx.x * d4 + c] = ab[i];
      }
    }
  }
  if (threadIdx.x == 0 && s_fail && dev_err != nullptr) atomicExch(dev_err, 2001);
}

// ---------------------------------------------------------------- backward, any d / alignment ---
__global__ void __launch_bounds__(LN_THREADS)
ln_bwd_generic_kernel(const float* __restrict__ x, const float* __restrict__ gamma,
                      const float* __restrict__ beta, const float* __restrict__ mean,
                      const float* __restrict__ rstd, const float* __restrict__ dy, float* __restrict__ dx,
                      float* __restrict__ part_dg, float* __restrict__ part_db, int64_t d, int64_t n, int act) {
  __shared__ float sh[64];
  float* pg = part_dg ? part_dg + (int64_t)blockIdx.x * d : nullptr;
  float* pb = part_db ? part_db + (int64_t)blockIdx.x * d : nullptr;
  if (pg)
    for (int64_t c = threadIdx.x; c < d; c += LN_THREADS) { pg[c] = 0.0f; pb[c] = 0.0f; }
  for (int64_t row = blockIdx.x; row < n; row += gridDim.x) {
    const float mu = mean[row], rs = rstd[row];
    const float* xr = x + row * d;
    const float* dyr = dy + row * d;
    float s1 = 0.0f, s2 = 0.0f;
    for (int64_t c = threadIdx.x; c < d; c += LN_THREADS) {
      const float xh = (xr[c] - mu) * rs;
      const float ga = gamma ? gamma[c] : 1.0f, be = beta ? beta[c] : 0.0f;
      const float dz = dyr[c] * fb_act_grad_z(act, fmaf(xh, ga, be));
      const float g = dz * ga;
      s1 += g;
      s2 += g * xh;
    }
    block_sum2(s1, s2, sh);
    const float m1 = s1 / (float)d, m2 = s2 / (float)d;
    float* dxr = dx + row * d;
    for (int64_t c = threadIdx.x; c < d; c += LN_THREADS) {
      const float xh = (xr[c] - mu) * rs;
      const float ga = gamma ? gamma[c] : 1.0f, be = beta ? beta[c] : 0.0f;
      const float dz = dyr[c] * fb_act_grad_z(act, fmaf(xh, ga, be));
      dxr[c] = rs * (dz * ga - m1 - xh * m2);
      if (pg) { pg[c] += dz * xh; pb[c] += dz; }   // column c is always owned by this thread
    }
  }
}

}  // namespace

// out_a[j] = sum_g part_a[g][j], out_b[j] = sum_g part_b[g][j]; block = 32 columns x 8 row groups.
__global__ void __launch_bounds__(256)
fb_colreduce2_kernel(const float* __restrict__ part_a, const float* __restrict__ part_b,
                     float* __restrict__ out_a, float* __restrict__ out_b, int64_t groups, int64_t d) {
  __shared__ float sa[8][33], sb[8][33];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const int64_t col = (int64_t)blockIdx.x * 32 + tx;
  float a = 0.0f, b = 0.0f;
  if (col < d) {
    // four independent loads per array in flight
    int64_t g = ty;
    for (; g + 24 < groups; g += 32) {
      const float a0 = part_a[g * d + col], a1 = part_a[(g + 8) * d + col], a2 = part_a[(g + 16) * d + col], a3 = part_a[(g + 24) * d + col];
      float b0 = 0.f, b1 = 0.f, b2 = 0.f, b3 = 0.f;
      if (part_b) { b0 = part_b[g * d + col]; b1 = part_b[(g + 8) * d + col]; b2 = part_b[(g + 16) * d + col]; b3 = part_b[(g + 24) * d + col]; }
      a += (a0 + a1) + (a2 + a3);
      b += (b0 + b1) + (b2 + b3);
    }
    for (; g < groups; g += 8) {
      a += part_a[g * d + col];
      if (part_b) b += part_b[g * d + col];
    }
  }
  sa[ty][tx] = a;
  sb[ty][tx] = b;
  __syncthreads();
  if (ty == 0 && col < d) {
#pragma unroll
    for (int i = 1; i < 8; ++i) { a += sa[i][tx]; b += sb[i][tx]; }
    out_a[col] = a;
    if (out_b) out_b[col] = b;
  }
}

static int ln_pick_v(int64_t d4) {
  const int64_t per = (d4 + LN_THREADS - 1) / LN_THREADS;
  if (per <= 1) return 1;
  if (per <= 2) return 2;
  if (per <= 4) return 4;
  if (per <= 8) return 8;
  return 0;
}

FB_API int32_t fb_layernorm_fwd(fb_ctx* ctx, void* stream_, const float* x, const float* gamma,
                                const float* beta, float* y, float* mean, float* rstd, int64_t d, int64_t n,
                                float eps, int32_t act) {
  FB_CHECK_CTX(ctx);
  cudaStream_t stream = (cudaStream_t)stream_;
  FB_REQUIRE(d >= 1 && n >= 0, FB_ERR_SHAPE, "fb_layernorm_fwd: bad shape d=%lld n=%lld", (long long)d, (long long)n);
  FB_REQUIRE(fb_act_valid(act), FB_ERR_INVALID_ARG, "fb_layernorm_fwd: unknown activation %d", act);
  FB_REQUIRE((gamma == nullptr) == (beta == nullptr), FB_ERR_INVALID_ARG, "fb_layernorm_fwd: gamma and beta must both be given or both NULL");
  if (n == 0) return FB_OK;
  FB_REQUIRE(x && y && mean && rstd, FB_ERR_INVALID_ARG, "fb_layernorm_fwd: NULL pointer");
  const bool vec = (d % 4 == 0) && fb_aligned16(x) && fb_aligned16(y) && (!gamma || (fb_aligned16(gamma) && fb_aligned16(beta)));
  const int v = vec ? ln_pick_v(d / 4) : 0;
  const unsigned grid = (unsigned)(n < (int64_t)ctx->sm_count * 64 ? n : (int64_t)ctx->sm_count * 64);
  if (v == 0) {
    ln_fwd_generic_kernel<<<grid, LN_THREADS, 0, stream>>>(x, gamma, beta, y, mean, rstd, d, n, eps, act);
  } else {
    const float4 *x4 = (const float4*)x, *g4 = (const float4*)gamma, *b4 = (const float4*)beta;
    float4* y4 = (float4*)y;
    const int d4 = (int)(d / 4);
    const unsigned gridv = (unsigned)(n < 0x7fffffff ? n : 0x7fffffff);
    switch (v) {
      case 1: ln_fwd_vec_kernel<1><<<gridv, LN_THREADS, 0, stream>>>(x4, g4, b4, y4, mean, rstd, d4, n, eps, act); break;
      case 2: ln_fwd_vec_kernel<2><<<gridv, LN_THREADS, 0, stream>>>(x4, g4, b4, y4, mean, rstd, d4, n, eps, act); break;
      case 4: ln_fwd_vec_kernel<4><<<gridv, LN_THREADS, 0, stream>>>(x4, g4, b4, y4, mean, rstd, d4, n, eps, act); break;
      default: ln_fwd_vec_kernel<8><<<gridv, LN_THREADS, 0, stream>>>(x4, g4, b4, y4, mean, rstd, d4, n, eps, act); break;
    }
  }
  FB_LAUNCH_CHECK();
  return FB_OK;
}

// Launches the backward kernels; `part` holds 2 * groups * d floats of per-block partials.
int32_t fb_layernorm_bwd_impl(cudaStream_t stream, int sm_count, float* part, int64_t groups, const float* x,
                              const float* gamma, const float* beta, const float* mean, const float* rstd,
                              const float* dy, float* dx, float* dgamma, float* dbeta, int64_t d, int64_t n,
                              int32_t act, int32_t* dev_err, bool allow_ring = true) {
  (void)sm_count;
  const bool want_param = (dgamma != nullptr);
  float* part_dg = want_param ? part : nullptr;
  float* part_db = want_param ? part + groups * d : nullptr;
  const bool vec = (d % 4 == 0) && fb_aligned16(x) && fb_aligned16(dy) && fb_aligned16(dx) &&
                   (!gamma || (fb_aligned16(gamma) && fb_aligned16(beta)));
  const int v = vec ? ln_pick_v(d / 4) : 0;
  if (v == 0) {
    ln_bwd_generic_kernel<<<(unsigned)groups, LN_THREADS, 0, stream>>>(x, gamma, beta, mean, rstd, dy, dx, part_dg,
                                                                       part_db, d, n, act);
  } else {
    const float4 *x4 = (const float4*)x, *g4 = (const float4*)gamma, *b4 = (const float4*)beta, *dy4 = (const float4*)dy;
    float4 *dx4 = (float4*)dx, *pg4 = (float4*)part_dg, *pb4 = (float4*)part_db;
    const int d4 = (int)(d / 4);
    const unsigned g = (unsigned)groups;
    // rows staged through shared memory when at least two stages of (x row, dy row) fit beside a second block
    const size_t stage_bytes = (size_t)2 * d * sizeof(float);
    int nst = (int)((size_t)100 * 1024 / stage_bytes);
    if (nst > LN_PIPE_MAX) nst = LN_PIPE_MAX;
    if (nst >= 2 && v >= 2 && allow_ring) {
      const size_t smem = (size_t)nst * stage_bytes;
      switch (v) {
        case 2:
          FB_CUDA(cudaFuncSetAttribute(ln_bwd_pipe_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
          ln_bwd_pipe_kernel<2><<<g, LN_THREADS, smem, stream>>>(x, g4, b4, mean, rstd, dy, dx4, pg4, pb4, d4, n, act, nst, dev_err);
          break;
        case 4:
          FB_CUDA(cudaFuncSetAttribute(ln_bwd_pipe_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
          ln_bwd_pipe_kernel<4><<<g, LN_THREADS, smem, stream>>>(x, g4, b4, mean, rstd, dy, dx4, pg4, pb4, d4, n, act, nst, dev_err);
          break;
        default:
          FB_CUDA(cudaFuncSetAttribute(ln_bwd_pipe_kernel<8>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
          ln_bwd_pipe_kernel<8><<<g, LN_THREADS, smem, stream>>>(x, g4, b4, mean, rstd, dy, dx4, pg4, pb4, d4, n, act, nst, dev_err);
          break;
      }
    } else {
      switch (v) {
        case 1: ln_bwd_vec_kernel<1><<<g, LN_THREADS, 0, stream>>>(x4, g4, b4, mean, rstd, dy4, dx4, pg4, pb4, d4, n, act); break;
        case 2: ln_bwd_vec_kernel<2><<<g, LN_THREADS, 0, stream>>>(x4, g4, b4, mean, rstd, dy4, dx4, pg4, pb4, d4, n, act); break;
        case 4: ln_bwd_vec_kernel<4><<<g, LN_THREADS, 0, stream>>>(x4, g4, b4, mean, rstd, dy4, dx4, pg4, pb4, d4, n, act); break;
        default: ln_bwd_vec_kernel<8><<<g, LN_THREADS, 0, stream>>>(x4, g4, b4, mean, rstd, dy4, dx4, pg4, pb4, d4, n, act); break;
      }
    }
  }
  FB_LAUNCH_CHECK();
  if (want_param) {
    fb_colreduce2_kernel<<<(unsigned)((d + 31) / 32), 256, 0, stream>>>(part_dg, part_db, dgamma, dbeta, groups, d);
    FB_LAUNCH_CHECK();
  }
  return FB_OK;
}

int64_t fb_layernorm_bwd_groups(int sm_count, int64_t n) {
  int64_t groups = (int64_t)sm_count * 2;
  if (groups > n) groups = n;
  if (groups < 1) groups = 1;
  return groups;
}

FB_API int32_t fb_layernorm_bwd(fb_ctx* ctx, void* stream_, const float* x, const float* gamma,
                                const float* beta, const float* mean, const float* rstd, const float* dy,
                                float* dx, float* dgamma, float* dbeta, int64_t d, int64_t n, int32_t act) {
  FB_CHECK_CTX(ctx);
  cudaStream_t stream = (cudaStream_t)stream_;
  FB_REQUIRE(d >= 1 && n >= 0, FB_ERR_SHAPE, "fb_layernorm_bwd: bad shape d=%lld n=%lld", (long long)d, (long long)n);
  FB_REQUIRE(fb_act_valid(act), FB_ERR_INVALID_ARG, "fb_layernorm_bwd: unknown activation %d", act);
  FB_REQUIRE((gamma == nullptr) == (beta == nullptr), FB_ERR_INVALID_ARG, "fb_layernorm_bwd: gamma and beta must both be given or both NULL");
  FB_REQUIRE((dgamma == nullptr) == (dbeta == nullptr), FB_ERR_INVALID_ARG, "fb_layernorm_bwd: dgamma and dbeta must both be given or both NULL");
  if (n == 0) {
    if (dgamma) {
      FB_CUDA(cudaMemsetAsync(dgamma, 0, d * sizeof(float), stream));
      FB_CUDA(cudaMemsetAsync(dbeta, 0, d * sizeof(float), stream));
    }
    return FB_OK;
  }
  FB_REQUIRE(x && mean && rstd && dy && dx, FB_ERR_INVALID_ARG, "fb_layernorm_bwd: NULL pointer");
  const int64_t groups = fb_layernorm_bwd_groups(ctx->sm_count, n);
  float* part = nullptr;
  if (dgamma) {
    part = (float*)fb_scratch(ctx, stream, (size_t)(2 * groups * d) * sizeof(float));
    if (!part) return FB_ERR_ALLOC;
  }
  return fb_layernorm_bwd_impl(stream, ctx->sm_count, part, groups, x, gamma, beta, mean, rstd, dy, dx, dgamma, dbeta,
                               d, n, act, ctx->dev_error);
}

// ------------------------------------------------------------- LayerNorm backward without allocation ---
// Some callers of this library may not allocate device memory at all: a serving or training process whose whole
// memory budget was handed out at start-up, code running between the begin and end of a stream capture (where an
// allocation is an error), or a host runtime whose finaliser / callback threads must not trigger the implicit
// device synchronisation that cudaMalloc and cudaFree can cause.  For them the per-block dgamma / dbeta partials
// of the backward pass live in the fixed array below instead of the context arena.
//
// The array is part of the library image: every GPU that loads the library holds these 16 MiB until the process
// exits.  Its name is only a host-side handle; the device address is looked up once per device with
// cudaGetSymbolAddress while that device is current, and that pointer is what the kernels receive.
#include <mutex>

constexpr int64_t FB_LN_STATIC_FLOATS = int64_t(4) << 20;   // 4 Mi floats = 16 MiB
static __device__ __align__(256) float g_ln_static_scratch[FB_LN_STATIC_FLOATS];

namespace {
struct LnStaticDevice {
  float* scratch = nullptr;   // device address of g_ln_static_scratch on this device
  int sm_count = 0;
  bool ready = false;
};
constexpr int LN_STATIC_MAX_DEVICES = 64;
LnStaticDevice g_ln_static_dev[LN_STATIC_MAX_DEVICES];
std::mutex g_ln_static_mutex;
}  // namespace

FB_API int32_t fb_layernorm_bwd_noalloc(void* stream_, const float* x, const float* gamma, const float* beta,
                                        const float* mean, const float* rstd, const float* dy, float* dx,
                                        float* dgamma, float* dbeta, int64_t d, int64_t n, int32_t act) {
  cudaStream_t stream = (cudaStream_t)stream_;
  FB_REQUIRE(d >= 1 && n >= 0, FB_ERR_SHAPE, "fb_layernorm_bwd_noalloc: bad shape d=%lld n=%lld", (long long)d, (long long)n);
  FB_REQUIRE(fb_act_valid(act), FB_ERR_INVALID_ARG, "fb_layernorm_bwd_noalloc: unknown activation %d", act);
  FB_REQUIRE((gamma == nullptr) == (beta == nullptr), FB_ERR_INVALID_ARG, "fb_layernorm_bwd_noalloc: gamma and beta must both be given or both NULL");
  FB_REQUIRE((dgamma == nullptr) == (dbeta == nullptr), FB_ERR_INVALID_ARG, "fb_layernorm_bwd_noalloc: dgamma and dbeta must both be given or both NULL");
  // the partials need 2 * groups * d floats with at least one group
  FB_REQUIRE(dgamma == nullptr || 2 * d <= FB_LN_STATIC_FLOATS, FB_ERR_UNSUPPORTED,
             "fb_layernorm_bwd_noalloc: d = %lld exceeds the fixed scratch (at most %lld features when dgamma/dbeta are "
             "requested); use fb_layernorm_bwd",
             (long long)d, (long long)(FB_LN_STATIC_FLOATS / 2));
  int dev = -1;
  FB_CUDA(cudaGetDevice(&dev));
  FB_REQUIRE(dev >= 0 && dev < LN_STATIC_MAX_DEVICES, FB_ERR_UNSUPPORTED, "fb_layernorm_bwd_noalloc: device index %d not supported", dev);
  LnStaticDevice& sd = g_ln_static_dev[dev];
  {
    // first call on this device: resolve the device address of the array (the device is current here)
    std::lock_guard<std::mutex> lock(g_ln_static_mutex);
    if (!sd.ready) {
      float* p = nullptr;
      FB_CUDA(cudaGetSymbolAddress((void**)&p, g_ln_static_scratch));
      int sms = 0;
      FB_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
      sd.scratch = p;
      sd.sm_count = sms;
      sd.ready = true;
    }
  }
  if (n == 0) {
    if (dgamma) {
      FB_CUDA(cudaMemsetAsync(dgamma, 0, d * sizeof(float), stream));
      FB_CUDA(cudaMemsetAsync(dbeta, 0, d * sizeof(float), stream));
    }
    return FB_OK;
  }
  FB_REQUIRE(x && mean && rstd && dy && dx, FB_ERR_INVALID_ARG, "fb_layernorm_bwd_noalloc: NULL pointer");
  int64_t groups = fb_layernorm_bwd_groups(sd.sm_count, n);
  if (dgamma != nullptr) {
    const int64_t fit = FB_LN_STATIC_FLOATS / (2 * d);   // >= 1 by the check above
    if (groups > fit) groups = fit;
  }
  // Every block overwrites all d columns of its own partial rows before the reduction reads exactly
  // groups * d of them, so nothing left behind by an earlier call is ever read.
  // This entry point has no context and therefore no device error word to report a timed-out wait through, so it
  // keeps to the kernels that hold their rows in registers and wait on nothing (no shared-memory ring).
  return fb_layernorm_bwd_impl(stream, sd.sm_count, sd.scratch, groups, x, gamma, beta, mean, rstd, dy, dx, dgamma, dbeta,
                               d, n, act, nullptr, /*allow_ring=*/false);
}
