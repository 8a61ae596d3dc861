// The rest of the layer family that sits on the same path as Dense / LayerNorm / BatchNorm / LSTM / GRU:
// GroupNorm and InstanceNorm, Embedding (gather / scatter-add), Dropout (counter-based random mask), and the
// RNNCell and GRUv3Cell time loops (built from the library's GEMM with fused accumulate + activation epilogue plus
// small gate kernels; one launch group per time step).
#include "common.cuh"

namespace {

constexpr int FT = 256;

__device__ __forceinline__ void block_sum2f(float& a, float& b, float* sh) {
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

// ------------------------------------------------------------------------------- GroupNorm ---
// x is [n][c][s]; row r = (sample, group) covers the L = (c / groups) * s contiguous floats that start at r * L.
__global__ void __launch_bounds__(FT)
gn_fwd_kernel(const float* __restrict__ x, const float* __restrict__ gamma, const float* __restrict__ beta,
              float* __restrict__ y, float* __restrict__ mean, float* __restrict__ rstd, int64_t s, int64_t cpg, int64_t groups,
              int64_t rows, float eps, int act) {
  __shared__ float sh[64];
  const int64_t L = cpg * s;
  for (int64_t r = blockIdx.x; r < rows; r += gridDim.x) {
    const float* xr = x + r * L;
    float a = 0.0f, zero = 0.0f;
    for (int64_t i = threadIdx.x; i < L; i += FT) a += xr[i];
    block_sum2f(a, zero, sh);
    const float mu = a / (float)L;
    float q = 0.0f;
    zero = 0.0f;
    for (int64_t i = threadIdx.x; i < L; i += FT) { const float d = xr[i] - mu; q += d * d; }
    block_sum2f(q, zero, sh);
    const float rs = rsqrtf(q / (float)L + eps);
    if (threadIdx.x == 0) { mean[r] = mu; rstd[r] = rs; }
    const int64_t c0 = (r % groups) * cpg;
    float* yr = y + r * L;
    for (int64_t i = threadIdx.x; i < L; i += FT) {
      float o = (xr[i] - mu) * rs;
      if (gamma != nullptr) { const int64_t c = c0 + i / s; o = fmaf(o, gamma[c], beta[c]); }
      yr[i] = fb_act_apply(act, o);
    }
  }
}

__global__ void __launch_bounds__(FT)
gn_bwd_dx_kernel(const float* __restrict__ x, const float* __restrict__ gamma, const float* __restrict__ beta,
                 const float* __restrict__ mean, const float* __restrict__ rstd, const float* __restrict__ dy,
                 float* __restrict__ dx, int64_t s, int64_t cpg, int64_t groups, int64_t rows, int act) {
  __shared__ float sh[64];
  const int64_t L = cpg * s;
  for (int64_t r = blockIdx.x; r < rows; r += gridDim.x) {
    const float mu = mean[r], rs = rstd[r];
    const float* xr = x + r * L;
    const float* dyr = dy + r * L;
    const int64_t c0 = (r % groups) * cpg;
    float s1 = 0.0f, s2 = 0.0f;
    for (int64_t i = threadIdx.x; i < L; i += FT) {
      const int64_t c = c0 + i / s;
      const float ga = gamma ? gamma[c] : 1.0f, be = beta ? beta[c] : 0.0f;
      const float xh = (xr[i] - mu) * rs;
      const float g = dyr[i] * fb_act_grad_z(act, fmaf(xh, ga, be)) * ga;
      s1 += g;
      s2 += g * xh;
    }
    block_sum2f(s1, s2, sh);
    const float m1 = s1 / (float)L, m2 = s2 / (float)L;
    float* dxr = dx + r * L;
    for (int64_t i = threadIdx.x; i < L; i += FT) {
      const int64_t c = c0 + i / s;
      const float ga = gamma ? gamma[c] : 1.0f, be = beta ? beta[c] : 0.0f;
      const float xh = (xr[i] - mu) * rs;
      const float g = dyr[i] * fb_act_grad_z(act, fmaf(xh, ga, be)) * ga;
      dxr[i] = rs * (g - m1 - xh * m2);
    }
  }
}

// dgamma[c] = sum over samples and positions of dz * xhat, dbeta[c] = sum of dz; one block per channel.
__global__ void __launch_bounds__(FT)
gn_bwd_param_kernel(const float* __restrict__ x, const float* __restrict__ gamma, const float* __restrict__ beta,
                    const float* __restrict__ mean, const float* __restrict__ rstd, const float* __restrict__ dy,
                    float* __restrict__ dgamma, float* __restrict__ dbeta, int64_t s, int64_t c_total, int64_t cpg,
                    int64_t groups, int64_t n, int act) {
  __shared__ float sh[64];
  const int64_t c = blockIdx.x;
  const int64_t g = c / cpg;
  const float ga = gamma[c], be = beta[c];
  float a = 0.0f, b = 0.0f;
  for (int64_t e = threadIdx.x; e < n * s; e += FT) {
    const int64_t smp = e / s, pos = e % s;
    const int64_t r = smp * groups + g;
    const int64_t off = (smp * c_total + c) * s + pos;
    const float xh = (x[off] - mean[r]) * rstd[r];
    const float dz = dy[off] * fb_act_grad_z(act, fmaf(xh, ga, be));
    a += dz * xh;
    b += dz;
  }
  block_sum2f(a, b, sh);
  if (threadIdx.x == 0) { dgamma[c] = a; dbeta[c] = b; }
}

// running statistics of InstanceNorm: averages over the samples of the per-(sample, channel) mean and variance
__global__ void __launch_bounds__(FT)
in_stats_kernel(const float* __restrict__ mean, const float* __restrict__ rstd, float* __restrict__ run_mean,
                float* __restrict__ run_var, int64_t c, int64_t n, float eps, float momentum, float corr) {
  const int64_t ch = (int64_t)blockIdx.x * FT + threadIdx.x;
  if (ch >= c) return;
  float m = 0.0f, v = 0.0f;
  for (int64_t i = 0; i < n; ++i) {
    m += mean[i * c + ch];
    const float rs = rstd[i * c + ch];
    v += 1.0f / (rs * rs) - eps;
  }
  m /= (float)n;
  v /= (float)n;
  run_mean[ch] = (1.0f - momentum) * run_mean[ch] + momentum * m;
  run_var[ch] = (1.0f - momentum) * run_var[ch] + momentum * corr * v;
}

// ------------------------------------------------------------------------------- Embedding ---
// y[:, i] = W[:, idx[i]] (1-based idx), zero where idx[i] == padding_idx; one warp per output column.
__global__ void __launch_bounds__(FT)
embedding_fwd_kernel(const float* __restrict__ W, const int32_t* __restrict__ idx, float* __restrict__ y, int64_t out_dim,
                     int64_t vocab, int64_t n, int32_t padding_idx, int32_t* __restrict__ dev_err) {
  const int lane = threadIdx.x & 31;
  const int64_t warp = ((int64_t)blockIdx.x * FT + threadIdx.x) >> 5, nwarps = ((int64_t)gridDim.x * FT) >> 5;
  for (int64_t i = warp; i < n; i += nwarps) {
    const int32_t id = idx[i];
    const bool bad = id < 1 || id > vocab;
    if (bad && lane == 0) atomicExch(dev_err, 5001);   // index outside 1:vocab (a BoundsError in the reference)
    const bool zero = bad || id == padding_idx;
    const float* src = W + (int64_t)(zero ? 0 : id - 1) * out_dim;
    float* dst = y + i * out_dim;
    for (int64_t j = lane; j < out_dim; j += 32) dst[j] = zero ? 0.0f : src[j];
  }
}

__global__ void __launch_bounds__(FT)
embedding_bwd_kernel(const float* __restrict__ dy, const int32_t* __restrict__ idx, float* __restrict__ dW, int64_t out_dim,
                     int64_t vocab, int64_t n, int32_t padding_idx) {
  const int lane = threadIdx.x & 31;
  const int64_t warp = ((int64_t)blockIdx.x * FT + threadIdx.x) >> 5, nwarps = ((int64_t)gridDim.x * FT) >> 5;
  for (int64_t i = warp; i < n; i += nwarps) {
    const int32_t id = idx[i];
    if (id < 1 || id > vocab || id == padding_idx) continue;
    float* dst = dW + (int64_t)(id - 1) * out_dim;
    const float* src = dy + i * out_dim;
    for (int64_t j = lane; j < out_dim; j += 32) atomicAdd(dst + j, src[j]);
  }
}

// --------------------------------------------------------------------------------- Dropout ---
// Philox4x32-10 (Salmon et al., "Parallel random numbers: as easy as 1, 2, 3"): counter = element index / 4 plus the
// caller's offset, key = the 64-bit seed.  Element i takes word i % 4 of its counter's output.
__global__ void __launch_bounds__(FT)
dropout_kernel(const float* __restrict__ x, float* __restrict__ y, int64_t count, float p, float scale, uint64_t seed,
               uint64_t offset) {
  const int64_t quads = (count + 3) / 4;
  for (int64_t q = (int64_t)blockIdx.x * FT + threadIdx.x; q < quads; q += (int64_t)gridDim.x * FT) {
    uint32_t r[4];
    philox4x32_10((uint64_t)q + offset, seed, r);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int64_t i = 4 * q + e;
      if (i < count) {
        const float u = (float)(r[e] >> 8) * (1.0f / 16777216.0f);   // uniform in [0, 1) with 24 bits
        y[i] = (u >= p) ? x[i] * scale : 0.0f;
      }
    }
  }
}

// --------------------------------------------------------------------- RNN / GRUv3 gate kernels ---
// All per-step arrays are [B] rows of H (or 3H) floats with a row stride: a time slice of a [B][T][.] array.

// G = D .* act'(y) (in place allowed), activations whose derivative follows from the output
__global__ void __launch_bounds__(FT)
rnn_bwd_gate_kernel(const float* __restrict__ d, int64_t ldd, const float* __restrict__ yv, int64_t ldy, float* __restrict__ g,
                    int64_t ldg, int H, int B, int act) {
  for (int64_t e = (int64_t)blockIdx.x * FT + threadIdx.x; e < (int64_t)B * H; e += (int64_t)gridDim.x * FT) {
    const int64_t b = e / H, j = e % H;
    g[b * ldg + j] = d[b * ldd + j] * fb_act_grad_y(act, yv[b * ldy + j]);
  }
}

// v = act(v) on B rows of H floats
__global__ void __launch_bounds__(FT) act_rows_kernel(float* __restrict__ v, int64_t ld, int H, int B, int act) {
  for (int64_t e = (int64_t)blockIdx.x * FT + threadIdx.x; e < (int64_t)B * H; e += (int64_t)gridDim.x * FT) {
    const int64_t b = e / H, j = e % H;
    v[b * ld + j] = fb_act_apply(act, v[b * ld + j]);
  }
}

// rh = r .* hprev (r = gates[:, 0:H])
__global__ void __launch_bounds__(FT)
gruv3_rh_kernel(const float* __restrict__ gates, int64_t ldg, const float* __restrict__ hprev, int64_t ldh,
                float* __restrict__ rh, int64_t ldr, int H, int B) {
  for (int64_t e = (int64_t)blockIdx.x * FT + threadIdx.x; e < (int64_t)B * H; e += (int64_t)gridDim.x * FT) {
    const int64_t b = e / H, j = e % H;
    const float hp = hprev ? hprev[b * ldh + j] : 0.0f;
    rh[b * ldr + j] = gates[b * ldg + j] * hp;
  }
}

// h' = (1 - z) .* htilde + z .* hprev
__global__ void __launch_bounds__(FT)
gruv3_out_kernel(const float* __restrict__ gates, int64_t ldg, const float* __restrict__ hprev, int64_t ldh,
                 float* __restrict__ out, int64_t ldo, float* __restrict__ hT, int H, int B) {
  for (int64_t e = (int64_t)blockIdx.x * FT + threadIdx.x; e < (int64_t)B * H; e += (int64_t)gridDim.x * FT) {
    const int64_t b = e / H, j = e % H;
    const float z = gates[b * ldg + H + j], ht = gates[b * ldg + 2 * H + j];
    const float hp = hprev ? hprev[b * ldh + j] : 0.0f;
    const float h = (1.0f - z) * ht + z * hp;
    out[b * ldo + j] = h;
    if (hT) hT[b * H + j] = h;
  }
}

// reverse, first half of a step: from dh (= d[:, t]) form the pre-activation cotangents of z and htilde and the
// direct path dh .* z
__global__ void __launch_bounds__(FT)
gruv3_bwd1_kernel(const float* __restrict__ d, int64_t ldd, const float* __restrict__ gates, int64_t ldg,
                  const float* __restrict__ hprev, int64_t ldh, float* __restrict__ g, int64_t ldgo,
                  float* __restrict__ direct, int H, int B) {
  for (int64_t e = (int64_t)blockIdx.x * FT + threadIdx.x; e < (int64_t)B * H; e += (int64_t)gridDim.x * FT) {
    const int64_t b = e / H, j = e % H;
    const float dh = d[b * ldd + j];
    const float z = gates[b * ldg + H + j], ht = gates[b * ldg + 2 * H + j];
    const float hp = hprev ? hprev[b * ldh + j] : 0.0f;
    g[b * ldgo + 2 * H + j] = dh * (1.0f - z) * (1.0f - ht * ht);
    g[b * ldgo + H + j] = dh * (hp - ht) * z * (1.0f - z);
    direct[b * H + j] = dh * z;
  }
}

// reverse, second half: drh = dpre3 * Wh_h (given); dpre1 = drh .* hprev .* r (1 - r); dprev += drh .* r + direct
__global__ void __launch_bounds__(FT)
gruv3_bwd2_kernel(const float* __restrict__ drh, const float* __restrict__ gates, int64_t ldg, const float* __restrict__ hprev,
                  int64_t ldh, const float* __restrict__ direct, float* __restrict__ g, int64_t ldgo, float* __restrict__ dprev,
                  int64_t ldp, int H, int B) {
  for (int64_t e = (int64_t)blockIdx.x * FT + threadIdx.x; e < (int64_t)B * H; e += (int64_t)gridDim.x * FT) {
    const int64_t b = e / H, j = e % H;
    const float r = gates[b * ldg + j];
    const float hp = hprev ? hprev[b * ldh + j] : 0.0f;
    const float v = drh[b * H + j];
    g[b * ldgo + j] = v * hp * r * (1.0f - r);
    if (dprev) dprev[b * ldp + j] += v * r + direct[b * H + j];
  }
}

// v[b][:] += w[b][:]
__global__ void __launch_bounds__(FT) add_rows_kernel(float* __restrict__ v, int64_t ldv, const float* __restrict__ w, int64_t ldw, int H, int B) {
  for (int64_t e = (int64_t)blockIdx.x * FT + threadIdx.x; e < (int64_t)B * H; e += (int64_t)gridDim.x * FT) {
    const int64_t b = e / H, j = e % H;
    v[b * ldv + j] += w[b * ldw + j];
  }
}

// dst[b][t][:] = src[b][t-1][:] for t >= 1, h0[b][:] (or zeros) for t = 0
__global__ void __launch_bounds__(FT)
shift_prev_h_kernel(const float* __restrict__ out, const float* __restrict__ h0, float* __restrict__ dst, int H, int64_t T,
                    int64_t B) {
  const int64_t total = B * T * H;
  for (int64_t e = (int64_t)blockIdx.x * FT + threadIdx.x; e < total; e += (int64_t)gridDim.x * FT) {
    const int64_t j = e % H, t = (e / H) % T, b = e / (H * T);
    dst[e] = t > 0 ? out[e - H] : (h0 ? h0[b * H + j] : 0.0f);
  }
}

__global__ void __launch_bounds__(FT) colsum_kernel(const float* __restrict__ a, float* __restrict__ out, int64_t rows, int64_t cols) {
  const int64_t c = (int64_t)blockIdx.x * FT + threadIdx.x;
  if (c >= cols) return;
  float s = 0.0f;
  for (int64_t r = 0; r < rows; ++r) s += a[r * cols + c];
  out[c] = s;
}

unsigned ew_grid(fb_ctx* ctx, int64_t work) {
  int64_t g = (work + FT - 1) / FT;
  const int64_t cap = (int64_t)ctx->sm_count * 8;
  if (g > cap) g = cap;
  return (unsigned)(g < 1 ? 1 : g);
}

int32_t check_norm_args(const char* fn, int64_t s, int64_t c, int64_t n, int64_t groups, int32_t act) {
  FB_REQUIRE(s >= 1 && c >= 1 && n >= 0 && groups >= 1, FB_ERR_SHAPE, "%s: bad shape s=%lld c=%lld n=%lld groups=%lld", fn, (long long)s,
             (long long)c, (long long)n, (long long)groups);
  FB_REQUIRE(c % groups == 0, FB_ERR_SHAPE, "%s: The number of groups (%lld) must divide the number of channels (%lld)", fn,
             (long long)groups, (long long)c);
  FB_REQUIRE(fb_act_valid(act), FB_ERR_INVALID_ARG, "%s: unknown activation %d", fn, act);
  return FB_OK;
}

}  // namespace

FB_API int32_t fb_groupnorm_fwd(fb_ctx* ctx, void* stream, const float* x, const float* gamma, const float* beta, float* y,
                                float* mean, float* rstd, int64_t s, int64_t c, int64_t n, int64_t groups, float eps, int32_t act) {
  FB_CHECK_CTX(ctx);
  int32_t st = check_norm_args("fb_groupnorm_fwd", s, c, n, groups, act);
  if (st != FB_OK) return st;
  FB_REQUIRE((gamma == nullptr) == (beta == nullptr), FB_ERR_INVALID_ARG, "fb_groupnorm_fwd: gamma and beta must both be given or both NULL");
  if (n == 0) return FB_OK;
  FB_REQUIRE(x && y && mean && rstd, FB_ERR_INVALID_ARG, "fb_groupnorm_fwd: NULL pointer");
  const int64_t rows = n * groups;
  const unsigned grid = (unsigned)(rows < (int64_t)ctx->sm_count * 8 ? rows : (int64_t)ctx->sm_count * 8);
  gn_fwd_kernel<<<grid, FT, 0, (cudaStream_t)stream>>>(x, gamma, beta, y, mean, rstd, s, c / groups, groups, rows, eps, act);
  FB_LAUNCH_CHECK();
  return FB_OK;
}

FB_API int32_t fb_groupnorm_bwd(fb_ctx* ctx, void* stream, const float* x, const float* gamma, const float* beta,
                                const float* mean, const float* rstd, const float* dy, float* dx, float* dgamma, float* dbeta,
                                int64_t s, int64_t c, int64_t n, int64_t groups, int32_t act) {
  FB_CHECK_CTX(ctx);
  int32_t st = check_norm_args("fb_groupnorm_bwd", s, c, n, groups, act);
  if (st != FB_OK) return st;
  FB_REQUIRE((gamma == nullptr) == (beta == nullptr), FB_ERR_INVALID_ARG, "fb_groupnorm_bwd: gamma and beta must both be given or both NULL");
  FB_REQUIRE((dgamma == nullptr) == (dbeta == nullptr), FB_ERR_INVALID_ARG, "fb_groupnorm_bwd: dgamma and dbeta must both be given or both NULL");
  FB_REQUIRE(dgamma == nullptr || gamma != nullptr, FB_ERR_INVALID_ARG, "fb_groupnorm_bwd: dgamma needs gamma");
  if (n == 0) {
    if (dgamma) {
      FB_CUDA(cudaMemsetAsync(dgamma, 0, c * sizeof(float), (cudaStream_t)stream));
      FB_CUDA(cudaMemsetAsync(dbeta, 0, c * sizeof(float), (cudaStream_t)stream));
    }
    return FB_OK;
  }
  FB_REQUIRE(x && mean && rstd && dy && dx, FB_ERR_INVALID_ARG, "fb_groupnorm_bwd: NULL pointer");
  const int64_t rows = n * groups;
  const unsigned grid = (unsigned)(rows < (int64_t)ctx->sm_count * 8 ? rows : (int64_t)ctx->sm_count * 8);
  gn_bwd_dx_kernel<<<grid, FT, 0, (cudaStream_t)stream>>>(x, gamma, beta, mean, rstd, dy, dx, s, c / groups, groups, rows, act);
  FB_LAUNCH_CHECK();
  if (dgamma) {
    gn_bwd_param_kernel<<<(unsigned)c, FT, 0, (cudaStream_t)stream>>>(x, gamma, beta, mean, rstd, dy, dgamma, dbeta, s, c, c / groups,
                                                                      groups, n, act);
    FB_LAUNCH_CHECK();
  }
  return FB_OK;
}

FB_API int32_t fb_instancenorm_update_stats(fb_ctx* ctx, void* stream, const float* mean, const float* rstd, float* running_mean,
                                            float* running_var, int64_t s, int64_t c, int64_t n, float eps, float momentum) {
  FB_CHECK_CTX(ctx);
  FB_REQUIRE(s >= 1 && c >= 1 && n >= 1, FB_ERR_SHAPE, "fb_instancenorm_update_stats: bad shape");
  FB_REQUIRE(mean && rstd && running_mean && running_var, FB_ERR_INVALID_ARG, "fb_instancenorm_update_stats: NULL pointer");
  const float corr = s > 1 ? (float)s / (float)(s - 1) : 1.0f;
  in_stats_kernel<<<(unsigned)((c + FT - 1) / FT), FT, 0, (cudaStream_t)stream>>>(mean, rstd, running_mean, running_var, c, n, eps,
                                                                                  momentum, corr);
  FB_LAUNCH_CHECK();
  return FB_OK;
}

FB_API int32_t fb_embedding_fwd(fb_ctx* ctx, void* stream, const float* W, const int32_t* idx, float* y, int64_t out_dim,
                                int64_t vocab, int64_t n, int32_t padding_idx) {
  FB_CHECK_CTX(ctx);
  FB_REQUIRE(out_dim >= 1 && vocab >= 1 && n >= 0, FB_ERR_SHAPE, "fb_embedding_fwd: bad shape");
  FB_REQUIRE(padding_idx >= 0 && padding_idx <= vocab, FB_ERR_INVALID_ARG, "fb_embedding_fwd: padding_idx=%d must be in 1:%lld", padding_idx,
             (long long)vocab);
  if (n == 0) return FB_OK;
  FB_REQUIRE(W && idx && y, FB_ERR_INVALID_ARG, "fb_embedding_fwd: NULL pointer");
  embedding_fwd_kernel<<<ew_grid(ctx, n * 32), FT, 0, (cudaStream_t)stream>>>(W, idx, y, out_dim, vocab, n, padding_idx, ctx->dev_error);
  FB_LAUNCH_CHECK();
  return FB_OK;
}

FB_API int32_t fb_embedding_bwd(fb_ctx* ctx, void* stream, const float* dy, const int32_t* idx, float* dW, int64_t out_dim,
                                int64_t vocab, int64_t n, int32_t padding_idx) {
  FB_CHECK_CTX(ctx);
  FB_REQUIRE(out_dim >= 1 && vocab >= 1 && n >= 0, FB_ERR_SHAPE, "fb_embedding_bwd: bad shape");
  FB_REQUIRE(dW, FB_ERR_INVALID_ARG, "fb_embedding_bwd: NULL pointer");
  FB_CUDA(cudaMemsetAsync(dW, 0, (size_t)(out_dim * vocab) * sizeof(float), (cudaStream_t)stream));
  if (n == 0) return FB_OK;
  FB_REQUIRE(dy && idx, FB_ERR_INVALID_ARG, "fb_embedding_bwd: NULL pointer");
  embedding_bwd_kernel<<<ew_grid(ctx, n * 32), FT, 0, (cudaStream_t)stream>>>(dy, idx, dW, out_dim, vocab, n, padding_idx);
  FB_LAUNCH_CHECK();
  return FB_OK;
}

FB_API int32_t fb_dropout(fb_ctx* ctx, void* stream, const float* x, float* y, int64_t count, float p, uint64_t seed, uint64_t offset) {
  FB_CHECK_CTX(ctx);
  FB_REQUIRE(count >= 0, FB_ERR_SHAPE, "fb_dropout: negative count");
  FB_REQUIRE(p >= 0.0f && p <= 1.0f, FB_ERR_INVALID_ARG, "fb_dropout: Dropout expects 0 <= p <= 1, got p = %g", (double)p);
  if (count == 0) return FB_OK;
  FB_REQUIRE(x && y, FB_ERR_INVALID_ARG, "fb_dropout: NULL pointer");
  const float scale = p < 1.0f ? 1.0f / (1.0f - p) : 0.0f;
  dropout_kernel<<<ew_grid(ctx, (count + 3) / 4), FT, 0, (cudaStream_t)stream>>>(x, y, count, p, scale, seed, offset);
  FB_LAUNCH_CHECK();
  return FB_OK;
}

// ----------------------------------------------------------------------------- RNNCell scan ---
namespace {
int32_t check_rnn_dims(const char* fn, int64_t in_dim, int64_t H, int64_t T, int64_t B) {
  FB_REQUIRE(in_dim >= 1 && H >= 1 && T >= 0 && B >= 0, FB_ERR_SHAPE, "%s: bad shape in=%lld hidden=%lld seq=%lld batch=%lld", fn,
             (long long)in_dim, (long long)H, (long long)T, (long long)B);
  FB_REQUIRE(H <= 0x3fffffff && B <= 0x3fffffff, FB_ERR_UNSUPPORTED, "%s: hidden size or batch too large", fn);
  return FB_OK;
}
fb_gemm_args plain_args() {
  fb_gemm_args a;
  memset(&a, 0, sizeof(a));
  a.act = FB_ACT_IDENTITY;
  return a;
}
}  // namespace

FB_API int64_t fb_rnn_cache_bytes(int64_t in_dim, int64_t hidden, int64_t seq_len, int64_t batch) {
  (void)in_dim;
  return 2 * seq_len * batch * hidden * (int64_t)sizeof(float);   // reverse-sweep cotangents, shifted outputs
}

FB_API int32_t fb_rnn_fwd(fb_ctx* ctx, void* stream_, int32_t act, const float* Wi, const float* Wh, const float* b, const float* x,
                          const float* h0, float* out, float* hT, int64_t in_dim, int64_t hidden, int64_t seq_len, int64_t batch) {
  FB_CHECK_CTX(ctx);
  cudaStream_t stream = (cudaStream_t)stream_;
  int32_t st = check_rnn_dims("fb_rnn_fwd", in_dim, hidden, seq_len, batch);
  if (st != FB_OK) return st;
  FB_REQUIRE(act == FB_ACT_IDENTITY || act == FB_ACT_RELU || act == FB_ACT_TANH || act == FB_ACT_SIGMOID, FB_ERR_UNSUPPORTED,
             "fb_rnn_fwd: activation %d has no recurrent kernel (identity, relu, tanh, sigmoid)", act);
  if (seq_len == 0 || batch == 0) return FB_OK;
  FB_REQUIRE(Wi && Wh && x && out, FB_ERR_INVALID_ARG, "fb_rnn_fwd: NULL pointer");
  const int64_t T = seq_len, rows = T * batch, H = hidden;
  // input projection of every step at once, written where the step's output will be
  fb_gemm_args a = plain_args();
  a.A = x; a.lda = in_dim; a.a_mn_major = 0;
  a.B = Wi; a.ldb = H; a.b_mn_major = 1;
  a.C = out; a.ldc = H; a.bias_n = b;
  a.M = rows; a.N = H; a.K = in_dim;
  st = fb_gemm_dispatch(ctx, stream, a, FB_PREC_DEFAULT);
  if (st != FB_OK) return st;
  for (int64_t t = 0; t < T; ++t) {
    float* out_t = out + t * H;
    if (t == 0 && h0 == nullptr) {
      // zero initial state: only the activation remains
      act_rows_kernel<<<ew_grid(ctx, batch * H), FT, 0, stream>>>(out_t, T * H, (int)H, (int)batch, act);
      FB_LAUNCH_CHECK();
      continue;
    }
    // out_t = act(out_t + hprev * Wh'): one GEMM with the accumulate + activation epilogue
    fb_gemm_args g = plain_args();
    g.A = t == 0 ? h0 : out + (t - 1) * H; g.lda = t == 0 ? H : T * H; g.a_mn_major = 0;
    g.B = Wh; g.ldb = H; g.b_mn_major = 1;
    g.C = out_t; g.ldc = T * H; g.M = batch; g.N = H; g.K = H; g.act = act; g.accumulate = 1;
    st = fb_gemm_dispatch(ctx, stream, g, FB_PREC_DEFAULT);
    if (st != FB_OK) return st;
  }
  if (hT) {
    FB_CUDA(cudaMemcpy2DAsync(hT, H * sizeof(float), out + (T - 1) * H, T * H * sizeof(float), H * sizeof(float), batch,
                              cudaMemcpyDeviceToDevice, stream));
  }
  return FB_OK;
}

// Reverse of fb_rnn_fwd.  `cache` (fb_rnn_cache_bytes) is scratch: [rows][H] cotangents, then [rows][H] shifted outputs.
FB_API int32_t fb_rnn_bwd(fb_ctx* ctx, void* stream_, int32_t act, const float* Wi, const float* Wh, const float* x, const float* h0,
                          const float* out, void* cache, const float* dout, const float* dhT, float* dWi, float* dWh, float* db,
                          float* dx, int64_t in_dim, int64_t hidden, int64_t seq_len, int64_t batch) {
  FB_CHECK_CTX(ctx);
  cudaStream_t stream = (cudaStream_t)stream_;
  int32_t st = check_rnn_dims("fb_rnn_bwd", in_dim, hidden, seq_len, batch);
  if (st != FB_OK) return st;
  FB_REQUIRE(seq_len >= 1 && batch >= 1, FB_ERR_SHAPE, "fb_rnn_bwd: empty sequence or batch");
  FB_REQUIRE(act == FB_ACT_IDENTITY || act == FB_ACT_RELU || act == FB_ACT_TANH || act == FB_ACT_SIGMOID, FB_ERR_UNSUPPORTED,
             "fb_rnn_bwd: activation %d has no recurrent kernel (identity, relu, tanh, sigmoid)", act);
  FB_REQUIRE(Wi && Wh && x && out && cache && dout && dWi && dWh, FB_ERR_INVALID_ARG, "fb_rnn_bwd: NULL pointer");
  const int64_t T = seq_len, rows = T * batch, H = hidden;
  float* G = (float*)cache;                 // starts as dout, ends as the pre-activation cotangents of every step
  float* hprev_all = G + rows * H;
  FB_CUDA(cudaMemcpyAsync(G, dout, (size_t)(rows * H) * sizeof(float), cudaMemcpyDeviceToDevice, stream));
  if (dhT) {
    // the final state is the last output: its cotangent joins dout[:, T]
    add_rows_kernel<<<ew_grid(ctx, batch * H), FT, 0, stream>>>(G + (T - 1) * H, T * H, dhT, H, (int)H, (int)batch);
    FB_LAUNCH_CHECK();
  }
  for (int64_t t = T - 1; t >= 0; --t) {
    float* g_t = G + t * H;
    rnn_bwd_gate_kernel<<<ew_grid(ctx, batch * H), FT, 0, stream>>>(g_t, T * H, out + t * H, T * H, g_t, T * H, (int)H, (int)batch, act);
    FB_LAUNCH_CHECK();
    if (t > 0) {
      // G[:, t-1] += g_t * Wh   (Wh is [H_out, H_in]: the operand indexed [in][out] is K-major with ld = H)
      fb_gemm_args g = plain_args();
      g.A = g_t; g.lda = T * H; g.a_mn_major = 0;
      g.B = Wh; g.ldb = H; g.b_mn_major = 0;
      g.C = G + (t - 1) * H; g.ldc = T * H; g.M = batch; g.N = H; g.K = H; g.accumulate = 1;
      st = fb_gemm_dispatch(ctx, stream, g, FB_PREC_DEFAULT);
      if (st != FB_OK) return st;
    }
  }
  shift_prev_h_kernel<<<ew_grid(ctx, rows * H), FT, 0, stream>>>(out, h0, hprev_all, (int)H, T, batch);
  FB_LAUNCH_CHECK();
  fb_gemm_args a = plain_args();
  a.A = x; a.lda = in_dim; a.a_mn_major = 1;
  a.B = G; a.ldb = H; a.b_mn_major = 1;
  a.C = dWi; a.ldc = H; a.M = in_dim; a.N = H; a.K = rows;
  st = fb_gemm_dispatch(ctx, stream, a, FB_PREC_DEFAULT);
  if (st != FB_OK) return st;
  a.A = hprev_all; a.lda = H; a.C = dWh; a.M = H;
  st = fb_gemm_dispatch(ctx, stream, a, FB_PREC_DEFAULT);
  if (st != FB_OK) return st;
  if (db) {
    colsum_kernel<<<(unsigned)((H + FT - 1) / FT), FT, 0, stream>>>(G, db, rows, H);
    FB_LAUNCH_CHECK();
  }
  if (dx) {
    a = plain_args();
    a.A = G; a.lda = H; a.a_mn_major = 0;
    a.B = Wi; a.ldb = H; a.b_mn_major = 0;
    a.C = dx; a.ldc = in_dim; a.M = rows; a.N = in_dim; a.K = H;
    st = fb_gemm_dispatch(ctx, stream, a, FB_PREC_DEFAULT);
  }
  return st;
}

// ---------------------------------------------------------------------------- GRUv3Cell scan ---
// cache layout: gates [rows][3H] (r, z, htilde after the forward pass), rh [rows][H] (r .* hprev); the reverse
// sweep adds D [rows][H] (running dh), G [rows][3H] (pre-activation cotangents), hprev_all [rows][H],
// drh [B][H] and direct [B][H].
FB_API int64_t fb_gruv3_cache_bytes(int64_t in_dim, int64_t hidden, int64_t seq_len, int64_t batch) {
  (void)in_dim;
  return (seq_len * batch * hidden * 9 + 2 * batch * hidden) * (int64_t)sizeof(float);
}

FB_API int32_t fb_gruv3_fwd(fb_ctx* ctx, void* stream_, const float* Wi, const float* Wh, const float* b, const float* Wh_h,
                            const float* x, const float* h0, float* out, float* hT, void* cache, int64_t in_dim, int64_t hidden,
                            int64_t seq_len, int64_t batch) {
  FB_CHECK_CTX(ctx);
  cudaStream_t stream = (cudaStream_t)stream_;
  int32_t st = check_rnn_dims("fb_gruv3_fwd", in_dim, hidden, seq_len, batch);
  if (st != FB_OK) return st;
  if (seq_len == 0 || batch == 0) return FB_OK;
  FB_REQUIRE(Wi && Wh && Wh_h && x && out, FB_ERR_INVALID_ARG, "fb_gruv3_fwd: NULL pointer");
  const int64_t T = seq_len, rows = T * batch, H = hidden;
  float* gates;
  float* rh;
  if (cache) {
    gates = (float*)cache;
    rh = gates + rows * 3 * H;
  } else {
    gates = (float*)fb_scratch(ctx, stream, (size_t)(rows * 4 * H) * sizeof(float));
    if (!gates) return FB_ERR_ALLOC;
    rh = gates + rows * 3 * H;
  }
  fb_gemm_args a = plain_args();
  a.A = x; a.lda = in_dim; a.a_mn_major = 0;
  a.B = Wi; a.ldb = 3 * H; a.b_mn_major = 1;
  a.C = gates; a.ldc = 3 * H; a.bias_n = b;
  a.M = rows; a.N = 3 * H; a.K = in_dim;
  st = fb_gemm_dispatch(ctx, stream, a, FB_PREC_DEFAULT);
  if (st != FB_OK) return st;
  const unsigned eg = ew_grid(ctx, batch * H);
  for (int64_t t = 0; t < T; ++t) {
    float* g_t = gates + t * 3 * H;
    const float* hprev = t == 0 ? h0 : out + (t - 1) * H;
    const int64_t ldh = t == 0 ? H : T * H;
    // r, z = sigmoid(gx12 + hprev * Wh12')
    if (hprev != nullptr) {
      fb_gemm_args g = plain_args();
      g.A = hprev; g.lda = ldh; g.a_mn_major = 0;
      g.B = Wh; g.ldb = 3 * H; g.b_mn_major = 1;
      g.C = g_t; g.ldc = T * 3 * H; g.M = batch; g.N = 2 * H; g.K = H; g.act = FB_ACT_SIGMOID; g.accumulate = 1;
      st = fb_gemm_dispatch(ctx, stream, g, FB_PREC_DEFAULT);
      if (st != FB_OK) return st;
    } else {
      act_rows_kernel<<<ew_grid(ctx, batch * 2 * H), FT, 0, stream>>>(g_t, T * 3 * H, (int)(2 * H), (int)batch, FB_ACT_SIGMOID);
      FB_LAUNCH_CHECK();
    }
    float* rh_t = rh + t * H;
    gruv3_rh_kernel<<<eg, FT, 0, stream>>>(g_t, T * 3 * H, hprev, ldh, rh_t, T * H, (int)H, (int)batch);
    FB_LAUNCH_CHECK();
    // htilde = tanh(gx3 + (r .* hprev) * Wh_h')
    if (hprev != nullptr) {
      fb_gemm_args g = plain_args();
      g.A = rh_t; g.lda = T * H; g.a_mn_major = 0;
      g.B = Wh_h; g.ldb = H; g.b_mn_major = 1;
      g.C = g_t + 2 * H; g.ldc = T * 3 * H; g.M = batch; g.N = H; g.K = H; g.act = FB_ACT_TANH; g.accumulate = 1;
      st = fb_gemm_dispatch(ctx, stream, g, FB_PREC_DEFAULT);
      if (st != FB_OK) return st;
    } else {
      act_rows_kernel<<<eg, FT, 0, stream>>>(g_t + 2 * H, T * 3 * H, (int)H, (int)batch, FB_ACT_TANH);
      FB_LAUNCH_CHECK();
    }
    gruv3_out_kernel<<<eg, FT, 0, stream>>>(g_t, T * 3 * H, hprev, ldh, out + t * H, T * H, t == T - 1 ? hT : nullptr, (int)H, (int)batch);
    FB_LAUNCH_CHECK();
  }
  return FB_OK;
}

FB_API int32_t fb_gruv3_bwd(fb_ctx* ctx, void* stream_, const float* Wi, const float* Wh, const float* Wh_h, const float* x,
                            const float* h0, const float* out, void* cache, const float* dout, const float* dhT, float* dWi,
                            float* dWh, float* db, float* dWh_h, float* dx, int64_t in_dim, int64_t hidden, int64_t seq_len,
                            int64_t batch) {
  FB_CHECK_CTX(ctx);
  cudaStream_t stream = (cudaStream_t)stream_;
  int32_t st = check_rnn_dims("fb_gruv3_bwd", in_dim, hidden, seq_len, batch);
  if (st != FB_OK) return st;
  FB_REQUIRE(seq_len >= 1 && batch >= 1, FB_ERR_SHAPE, "fb_gruv3_bwd: empty sequence or batch");
  FB_REQUIRE(Wi && Wh && Wh_h && x && out && cache && dout && dWi && dWh && dWh_h, FB_ERR_INVALID_ARG, "fb_gruv3_bwd: NULL pointer");
  const int64_t T = seq_len, rows = T * batch, H = hidden;
  float* gates = (float*)cache;
  float* rh = gates + rows * 3 * H;
  float* D = rh + rows * H;
  float* G = D + rows * H;
  float* hprev_all = G + rows * 3 * H;
  float* drh = hprev_all + rows * H;
  float* direct = drh + batch * H;
  FB_CUDA(cudaMemcpyAsync(D, dout, (size_t)(rows * H) * sizeof(float), cudaMemcpyDeviceToDevice, stream));
  const unsigned eg = ew_grid(ctx, batch * H);
  if (dhT) {
    add_rows_kernel<<<eg, FT, 0, stream>>>(D + (T - 1) * H, T * H, dhT, H, (int)H, (int)batch);
    FB_LAUNCH_CHECK();
  }
  for (int64_t t = T - 1; t >= 0; --t) {
    const float* g_t = gates + t * 3 * H;
    float* G_t = G + t * 3 * H;
    const float* hprev = t == 0 ? h0 : out + (t - 1) * H;
    const int64_t ldh = t == 0 ? H : T * H;
    gruv3_bwd1_kernel<<<eg, FT, 0, stream>>>(D + t * H, T * H, g_t, T * 3 * H, hprev, ldh, G_t, T * 3 * H, direct, (int)H, (int)batch);
    FB_LAUNCH_CHECK();
    // drh = dpre3 * Wh_h  ([B][H_out] x [H_out, H_in])
    fb_gemm_args g = plain_args();
    g.A = G_t + 2 * H; g.lda = T * 3 * H; g.a_mn_major = 0;
    g.B = Wh_h; g.ldb = H; g.b_mn_major = 0;
    g.C = drh; g.ldc = H; g.M = batch; g.N = H; g.K = H;
    st = fb_gemm_dispatch(ctx, stream, g, FB_PREC_DEFAULT);
    if (st != FB_OK) return st;
    gruv3_bwd2_kernel<<<eg, FT, 0, stream>>>(drh, g_t, T * 3 * H, hprev, ldh, direct, G_t, T * 3 * H, t > 0 ? D + (t - 1) * H : nullptr,
                                             T * H, (int)H, (int)batch);
    FB_LAUNCH_CHECK();
    if (t > 0) {
      // D[:, t-1] += [dpre1, dpre2] * Wh12
      g = plain_args();
      g.A = G_t; g.lda = T * 3 * H; g.a_mn_major = 0;
      g.B = Wh; g.ldb = 3 * H; g.b_mn_major = 0;
      g.C = D + (t - 1) * H; g.ldc = T * H; g.M = batch; g.N = H; g.K = 2 * H; g.accumulate = 1;
      st = fb_gemm_dispatch(ctx, stream, g, FB_PREC_DEFAULT);
      if (st != FB_OK) return st;
    }
  }
  shift_prev_h_kernel<<<ew_grid(ctx, rows * H), FT, 0, stream>>>(out, h0, hprev_all, (int)H, T, batch);
  FB_LAUNCH_CHECK();
  fb_gemm_args a = plain_args();
  a.A = x; a.lda = in_dim; a.a_mn_major = 1;
  a.B = G; a.ldb = 3 * H; a.b_mn_major = 1;
  a.C = dWi; a.ldc = 3 * H; a.M = in_dim; a.N = 3 * H; a.K = rows;
  st = fb_gemm_dispatch(ctx, stream, a, FB_PREC_DEFAULT);
  if (st != FB_OK) return st;
  // dWh: only the r and z rows receive a gradient; the third block of Wh is never read by the cell (recurrent.jl:804)
  FB_CUDA(cudaMemsetAsync(dWh, 0, (size_t)(3 * H * H) * sizeof(float), stream));
  a.A = hprev_all; a.lda = H; a.C = dWh; a.M = H; a.N = 2 * H;
  st = fb_gemm_dispatch(ctx, stream, a, FB_PREC_DEFAULT);
  if (st != FB_OK) return st;
  // dWh_h = dpre3' * rh
  a = plain_args();
  a.A = rh; a.lda = H; a.a_mn_major = 1;
  a.B = G + 2 * H; a.ldb = 3 * H; a.b_mn_major = 1;
  a.C = dWh_h; a.ldc = H; a.M = H; a.N = H; a.K = rows;
  st = fb_gemm_dispatch(ctx, stream, a, FB_PREC_DEFAULT);
  if (st != FB_OK) return st;
  if (db) {
    colsum_kernel<<<(unsigned)((3 * H + FT - 1) / FT), FT, 0, stream>>>(G, db, rows, 3 * H);
    FB_LAUNCH_CHECK();
  }
  if (dx) {
    a = plain_args();
    a.A = G; a.lda = 3 * H; a.a_mn_major = 0;
    a.B = Wi; a.ldb = 3 * H; a.b_mn_major = 0;
    a.C = dx; a.ldc = in_dim; a.M = rows; a.N = in_dim; a.K = 3 * H;
    st = fb_gemm_dispatch(ctx, stream, a, FB_PREC_DEFAULT);
  }
  return st;
}
