// The bf16 entry points of the Dense path (Flux.bf16, src/functor.jl:274): matmul and Dense forward / backward with
// BFloat16 storage for weights, activations and gradients, fp32 accumulation on the tensor cores (gemm_bf16.cu).
//
// Row-major views of Julia's column-major arrays, as in dense.cu:
//   forward   Y[n][out]    = X[n][in]    * Wm[in][out]        (A K-major,  B MN-major, bias along out)
//   dX        dX[n][in]    = D[n][out]   * Wm[in][out]^T      (A K-major,  B K-major)
//   dW        dWm[in][out] = X[n][in]^T  * D[n][out]          (A MN-major, B MN-major)
#include <cuda_bf16.h>

#include "common.cuh"

namespace {

__device__ __forceinline__ float bf2f(uint16_t v) { return __uint_as_float((uint32_t)v << 16); }
__device__ __forceinline__ uint16_t f2bf(float v) {
  const __nv_bfloat16 b = __float2bfloat16_rn(v);
  return *reinterpret_cast<const uint16_t*>(&b);
}

// delta = dy .* act'(.) (bf16) and per-block partial column sums of delta (fp32): block (x: 64 columns, y: row group)
__global__ void __launch_bounds__(256)
act_bwd_colsum_bf16_kernel(int act, const uint16_t* __restrict__ dy, const uint16_t* __restrict__ y, const uint16_t* __restrict__ z,
                           uint16_t* __restrict__ delta, float* __restrict__ part, int64_t rows, int64_t cols, int64_t rpb) {
  __shared__ float sh[4][64];
  const int tx = threadIdx.x & 63, ty = threadIdx.x >> 6;
  const int64_t col = (int64_t)blockIdx.x * 64 + tx;
  const int64_t r0 = (int64_t)blockIdx.y * rpb, r1 = (r0 + rpb < rows) ? r0 + rpb : rows;
  float s = 0.0f;
  if (col < cols) {
    for (int64_t r = r0 + ty; r < r1; r += 4) {
      const int64_t i = r * cols + col;
      float d = bf2f(dy[i]);
      if (act != FB_ACT_IDENTITY) {
        d *= (act == FB_ACT_GELU_TANH || act == FB_ACT_GELU_ERF) ? fb_act_grad_z(act, bf2f(z[i])) : fb_act_grad_y(act, bf2f(y[i]));
        const uint16_t q = f2bf(d);
        delta[i] = q;
        d = bf2f(q);          // the bias gradient sums what the GEMMs will read
      }
      s += d;
    }
  }
  sh[ty][tx] = s;
  __syncthreads();
  if (ty == 0 && col < cols && part != nullptr) part[(int64_t)blockIdx.y * cols + col] = (sh[0][tx] + sh[1][tx]) + (sh[2][tx] + sh[3][tx]);
}

__global__ void __launch_bounds__(256) colsum_parts_bf16_kernel(const float* __restrict__ part, uint16_t* __restrict__ out, int64_t groups, int64_t cols) {
  const int64_t c = (int64_t)blockIdx.x * 256 + threadIdx.x;
  if (c >= cols) return;
  float s = 0.0f;
  for (int64_t g = 0; g < groups; ++g) s += part[g * cols + c];
  out[c] = f2bf(s);
}

__global__ void __launch_bounds__(256) axpy_bf16_kernel(float alpha, const uint16_t* __restrict__ x, uint16_t* __restrict__ y, int64_t count) {
  for (int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x; i < count; i += (int64_t)gridDim.x * 256)
    y[i] = f2bf(fmaf(alpha, bf2f(x[i]), bf2f(y[i])));
}

}  // namespace

FB_API int32_t fb_axpy_bf16(fb_ctx* ctx, void* stream, float alpha, const uint16_t* x, uint16_t* y, int64_t count) {
  FB_CHECK_CTX(ctx);
  FB_REQUIRE(count >= 0, FB_ERR_INVALID_ARG, "fb_axpy_bf16: negative count");
  if (count == 0) return FB_OK;
  FB_REQUIRE(x && y, FB_ERR_INVALID_ARG, "fb_axpy_bf16: NULL pointer");
  int64_t blocks = (count + 255) / 256;
  if (blocks > (int64_t)ctx->sm_count * 16) blocks = (int64_t)ctx->sm_count * 16;
  axpy_bf16_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(alpha, x, y, count);
  FB_LAUNCH_CHECK();
  return FB_OK;
}

FB_API int32_t fb_gemm_bf16(fb_ctx* ctx, void* stream, int32_t transa, int32_t transb, int64_t m, int64_t n, int64_t k,
                            const uint16_t* A, int64_t lda, const uint16_t* B, int64_t ldb, void* C, int64_t ldc,
                            int32_t accumulate, int32_t c_is_f32) {
  FB_CHECK_CTX(ctx);
  FB_REQUIRE(m >= 0 && n >= 0 && k >= 0, FB_ERR_SHAPE, "fb_gemm_bf16: negative dimension");
  FB_REQUIRE((transa == 0 || transa == 1) && (transb == 0 || transb == 1), FB_ERR_INVALID_ARG, "fb_gemm_bf16: trans flags must be 0 or 1");
  if (m == 0 || n == 0) return FB_OK;
  FB_REQUIRE(k >= 1, FB_ERR_SHAPE, "fb_gemm_bf16: k must be at least 1");
  FB_REQUIRE(A && B && C, FB_ERR_INVALID_ARG, "fb_gemm_bf16: NULL pointer");
  FB_REQUIRE(lda >= (transa ? k : m) && ldb >= (transb ? n : k) && ldc >= m, FB_ERR_SHAPE, "fb_gemm_bf16: leading dimension too small");
  // column-major C[m,n] is the row-major C'[n][m] = op(B)^T * op(A)^T
  fb_gemm_bf16_args a;
  a.A = B; a.lda = ldb; a.a_mn_major = transb ? 1 : 0;
  a.B = A; a.ldb = lda; a.b_mn_major = transa ? 0 : 1;
  a.C = C; a.ldc = ldc; a.Z = nullptr; a.bias_n = nullptr;
  a.M = n; a.N = m; a.K = k; a.act = FB_ACT_IDENTITY; a.accumulate = accumulate ? 1 : 0; a.out_f32 = c_is_f32 ? 1 : 0;
  return fb_gemm_bf16_launch(ctx, (cudaStream_t)stream, a);
}

FB_API int32_t fb_dense_fwd_bf16(fb_ctx* ctx, void* stream, int32_t act, const uint16_t* W, const uint16_t* b, const uint16_t* x,
                                 uint16_t* y, uint16_t* z, int64_t out_dim, int64_t in_dim, int64_t n) {
  FB_CHECK_CTX(ctx);
  FB_REQUIRE(out_dim >= 1 && in_dim >= 1 && n >= 0, FB_ERR_SHAPE, "fb_dense_fwd_bf16: bad shape out=%lld in=%lld n=%lld",
             (long long)out_dim, (long long)in_dim, (long long)n);
  FB_REQUIRE(fb_act_valid(act), FB_ERR_INVALID_ARG, "fb_dense_fwd_bf16: unknown activation %d", act);
  if (n == 0) return FB_OK;
  FB_REQUIRE(W && x && y, FB_ERR_INVALID_ARG, "fb_dense_fwd_bf16: NULL pointer");
  fb_gemm_bf16_args a;
  a.A = x; a.lda = in_dim; a.a_mn_major = 0;
  a.B = W; a.ldb = out_dim; a.b_mn_major = 1;
  a.C = y; a.ldc = out_dim; a.Z = z; a.bias_n = b;
  a.M = n; a.N = out_dim; a.K = in_dim; a.act = act; a.accumulate = 0; a.out_f32 = 0;
  return fb_gemm_bf16_launch(ctx, (cudaStream_t)stream, a);
}

FB_API int32_t fb_dense_bwd_bf16(fb_ctx* ctx, void* stream_, int32_t act, const uint16_t* W, const uint16_t* x, const uint16_t* y,
                                 const uint16_t* z, const uint16_t* dy, uint16_t* delta, uint16_t* dW, uint16_t* db, uint16_t* dx,
                                 int64_t out_dim, int64_t in_dim, int64_t n) {
  FB_CHECK_CTX(ctx);
  cudaStream_t stream = (cudaStream_t)stream_;
  FB_REQUIRE(out_dim >= 1 && in_dim >= 1 && n >= 1, FB_ERR_SHAPE, "fb_dense_bwd_bf16: bad shape out=%lld in=%lld n=%lld",
             (long long)out_dim, (long long)in_dim, (long long)n);
  FB_REQUIRE(fb_act_valid(act), FB_ERR_INVALID_ARG, "fb_dense_bwd_bf16: unknown activation %d", act);
  FB_REQUIRE(W && x && dy && dW, FB_ERR_INVALID_ARG, "fb_dense_bwd_bf16: NULL pointer");
  const bool need_delta = (act != FB_ACT_IDENTITY);
  if (need_delta) {
    FB_REQUIRE(delta != nullptr, FB_ERR_INVALID_ARG, "fb_dense_bwd_bf16: delta scratch is required for a non-identity activation");
    if (fb_act_needs_z(act)) FB_REQUIRE(z != nullptr, FB_ERR_INVALID_ARG, "fb_dense_bwd_bf16: the gelu activations need the saved pre-activation z");
    else FB_REQUIRE(y != nullptr, FB_ERR_INVALID_ARG, "fb_dense_bwd_bf16: the forward output y is required");
  }
  if (need_delta || db != nullptr) {
    const int64_t gx = (out_dim + 63) / 64;
    int64_t gy = ((int64_t)ctx->sm_count * 4 + gx - 1) / gx;
    if (gy > (n + 3) / 4) gy = (n + 3) / 4;
    if (gy < 1) gy = 1;
    if (gy > 65535) gy = 65535;
    const int64_t rpb = (n + gy - 1) / gy;
    gy = (n + rpb - 1) / rpb;
    float* part = nullptr;
    if (db != nullptr) {
      part = (float*)fb_scratch(ctx, stream, (size_t)(gy * out_dim) * sizeof(float));
      if (!part) return FB_ERR_ALLOC;
    }
    act_bwd_colsum_bf16_kernel<<<dim3((unsigned)gx, (unsigned)gy), 256, 0, stream>>>(act, dy, y, z, need_delta ? delta : nullptr, part, n,
                                                                                    out_dim, rpb);
    FB_LAUNCH_CHECK();
    if (db != nullptr) {
      colsum_parts_bf16_kernel<<<(unsigned)((out_dim + 255) / 256), 256, 0, stream>>>(part, db, gy, out_dim);
      FB_LAUNCH_CHECK();
    }
  }
  const uint16_t* D = need_delta ? delta : dy;
  fb_gemm_bf16_args a;
  a.Z = nullptr; a.bias_n = nullptr; a.act = FB_ACT_IDENTITY; a.accumulate = 0; a.out_f32 = 0;
  a.A = x; a.lda = in_dim; a.a_mn_major = 1;
  a.B = D; a.ldb = out_dim; a.b_mn_major = 1;
  a.C = dW; a.ldc = out_dim; a.M = in_dim; a.N = out_dim; a.K = n;
  int32_t st = fb_gemm_bf16_launch(ctx, stream, a);
  if (st != FB_OK) return st;
  if (dx != nullptr) {
    a.A = D; a.lda = out_dim; a.a_mn_major = 0;
    a.B = W; a.ldb = out_dim; a.b_mn_major = 0;
    a.C = dx; a.ldc = in_dim; a.M = n; a.N = in_dim; a.K = out_dim;
    st = fb_gemm_bf16_launch(ctx, stream, a);
  }
  return st;
}
