// Matmul dispatch and the Dense layer entry points.
//
// All matrices reach the kernels as row-major views of Julia's column-major arrays:
//   forward   Y[n][out]  = X[n][in]   * Wm[in][out]          (A K-major,  B MN-major, bias along out)
//   dX        dX[n][in]  = D[n][out]  * Wm[in][out]^T        (A K-major,  B K-major)
//   dW        dWm[in][out] = X[n][in]^T * D[n][out]          (A MN-major, B MN-major)
// where Wm is the memory of Julia's W[out, in].
#include "common.cuh"

#include <stdlib.h>

// FLUXB200_PRECISION = fp32_simt | 3xtf32 | tf32 replaces FB_PREC_DEFAULT (read once per process).
static int default_precision_override() {
  static int cached = -1;
  if (cached < 0) {
    cached = FB_PREC_DEFAULT;
    const char* e = getenv("FLUXB200_PRECISION");
    if (e != nullptr) {
      if (strcmp(e, "fp32_simt") == 0) cached = FB_PREC_FP32_SIMT;
      else if (strcmp(e, "3xtf32") == 0) cached = FB_PREC_DEFAULT;
      else if (strcmp(e, "tf32") == 0) cached = FB_PREC_TF32;
    }
  }
  return cached;
}

int32_t fb_gemm_dispatch(fb_ctx* ctx, cudaStream_t stream, const fb_gemm_args& a, int precision) {
  if (a.M == 0 || a.N == 0) return FB_OK;
  if (precision == FB_PREC_DEFAULT) {
    const int o = default_precision_override();
    if (o == FB_PREC_FP32_SIMT) precision = o;
    else if (o == FB_PREC_TF32 && fb_gemm_tc_supported(a)) precision = o;
  }
  switch (precision) {
    case FB_PREC_FP32_SIMT:
      return fb_gemm_simt_launch(ctx, stream, a);
    case FB_PREC_3XTF32:
    case FB_PREC_3XTF32_PAIR:
    case FB_PREC_TF32: {
      const int32_t st = fb_gemm_tc_launch(ctx, stream, a, precision == FB_PREC_TF32 ? 1 : precision == FB_PREC_3XTF32 ? 3 : 32);
      if (st == FB_ERR_UNSUPPORTED)
        return fb_fail(FB_ERR_UNSUPPORTED,
                       "gemm: the tensor-core kernel needs 16-byte aligned pointers, leading dimensions that are "
                       "multiples of 4 and K >= 1 (M=%lld N=%lld K=%lld lda=%lld ldb=%lld ldc=%lld)",
                       (long long)a.M, (long long)a.N, (long long)a.K, (long long)a.lda, (long long)a.ldb, (long long)a.ldc);
      return st;
    }
    case FB_PREC_DEFAULT: {
      const bool big = (double)a.M * (double)a.N * (double)a.K >= 1048576.0 && a.K >= 32 && a.N >= 32;
      if (big && fb_gemm_tc_supported(a)) return fb_gemm_tc_launch(ctx, stream, a, 3);
      return fb_gemm_simt_launch(ctx, stream, a);
    }
    default:
      return fb_fail(FB_ERR_INVALID_ARG, "gemm: unknown precision %d", precision);
  }
}

FB_API int32_t fb_gemm_f32(fb_ctx* ctx, void* stream, int32_t transa, int32_t transb, int64_t m, int64_t n, int64_t k,
                           const float* A, int64_t lda, const float* B, int64_t ldb, float* C, int64_t ldc,
                           int32_t accumulate, int32_t precision) {
  FB_CHECK_CTX(ctx);
  FB_REQUIRE(m >= 0 && n >= 0 && k >= 0, FB_ERR_SHAPE, "fb_gemm_f32: negative dimension");
  FB_REQUIRE((transa == 0 || transa == 1) && (transb == 0 || transb == 1), FB_ERR_INVALID_ARG, "fb_gemm_f32: trans flags must be 0 or 1");
  if (m == 0 || n == 0) return FB_OK;
  FB_REQUIRE(A && B && C, FB_ERR_INVALID_ARG, "fb_gemm_f32: NULL pointer");
  FB_REQUIRE(lda >= (transa ? k : m) && ldb >= (transb ? n : k) && ldc >= m && lda >= 1 && ldb >= 1, FB_ERR_SHAPE,
             "fb_gemm_f32: leading dimension too small");
  // column-major C[m,n] is the row-major C'[n][m] = op(B)^T * op(A)^T
  fb_gemm_args a;
  a.A = B; a.lda = ldb; a.a_mn_major = transb ? 1 : 0;
  a.B = A; a.ldb = lda; a.b_mn_major = transa ? 0 : 1;
  a.C = C; a.ldc = ldc; a.Z = nullptr; a.bias_n = nullptr; a.bias_m = nullptr;
  a.M = n; a.N = m; a.K = k; a.act = FB_ACT_IDENTITY; a.accumulate = accumulate ? 1 : 0;
  return fb_gemm_dispatch(ctx, (cudaStream_t)stream, a, precision);
}

FB_API int32_t fb_dense_fwd(fb_ctx* ctx, void* stream, int32_t act, int32_t precision, const float* W, const float* b,
                            const float* x, float* y, float* z, int64_t out_dim, int64_t in_dim, int64_t n) {
  FB_CHECK_CTX(ctx);
  FB_REQUIRE(out_dim >= 1 && in_dim >= 1 && n >= 0, FB_ERR_SHAPE, "fb_dense_fwd: bad shape out=%lld in=%lld n=%lld",
             (long long)out_dim, (long long)in_dim, (long long)n);
  FB_REQUIRE(fb_act_valid(act), FB_ERR_INVALID_ARG, "fb_dense_fwd: unknown activation %d", act);
  if (n == 0) return FB_OK;
  FB_REQUIRE(W && x && y, FB_ERR_INVALID_ARG, "fb_dense_fwd: NULL pointer");
  fb_gemm_args a;
  a.A = x; a.lda = in_dim; a.a_mn_major = 0;
  a.B = W; a.ldb = out_dim; a.b_mn_major = 1;
  a.C = y; a.ldc = out_dim; a.Z = z; a.bias_n = b; a.bias_m = nullptr;
  a.M = n; a.N = out_dim; a.K = in_dim; a.act = act; a.accumulate = 0;
  return fb_gemm_dispatch(ctx, (cudaStream_t)stream, a, precision);
}

FB_API int32_t fb_dense_bwd(fb_ctx* ctx, void* stream_, int32_t act, int32_t precision, const float* W, const float* x,
                            const float* y, const float* z, const float* dy, float* delta, float* dW, float* db,
                            float* dx, int64_t out_dim, int64_t in_dim, int64_t n) {
  FB_CHECK_CTX(ctx);
  cudaStream_t stream = (cudaStream_t)stream_;
  FB_REQUIRE(out_dim >= 1 && in_dim >= 1 && n >= 0, FB_ERR_SHAPE, "fb_dense_bwd: bad shape out=%lld in=%lld n=%lld",
             (long long)out_dim, (long long)in_dim, (long long)n);
  FB_REQUIRE(fb_act_valid(act), FB_ERR_INVALID_ARG, "fb_dense_bwd: unknown activation %d", act);
  FB_REQUIRE(W && x && dy && dW, FB_ERR_INVALID_ARG, "fb_dense_bwd: NULL pointer");
  if (n == 0) {
    FB_CUDA(cudaMemsetAsync(dW, 0, (size_t)(out_dim * in_dim) * sizeof(float), stream));
    if (db) FB_CUDA(cudaMemsetAsync(db, 0, (size_t)out_dim * sizeof(float), stream));
    return FB_OK;
  }
  int32_t st = fb_act_bwd_colsum(ctx, stream, act, dy, y, z, delta, db, n, out_dim);
  if (st != FB_OK) return st;
  const float* D = (act == FB_ACT_IDENTITY) ? dy : delta;
  fb_gemm_args a;
  // dW: [in][out] = X^T * D
  a.A = x; a.lda = in_dim; a.a_mn_major = 1;
  a.B = D; a.ldb = out_dim; a.b_mn_major = 1;
  a.C = dW; a.ldc = out_dim; a.Z = nullptr; a.bias_n = nullptr; a.bias_m = nullptr;
  a.M = in_dim; a.N = out_dim; a.K = n; a.act = FB_ACT_IDENTITY; a.accumulate = 0;
  st = fb_gemm_dispatch(ctx, stream, a, precision);
  if (st != FB_OK) return st;
  if (dx != nullptr) {
    // dX: [n][in] = D * Wm^T
    a.A = D; a.lda = out_dim; a.a_mn_major = 0;
    a.B = W; a.ldb = out_dim; a.b_mn_major = 0;
    a.C = dx; a.ldc = in_dim;
    a.M = n; a.N = in_dim; a.K = out_dim;
    st = fb_gemm_dispatch(ctx, stream, a, precision);
  }
  return st;
}
