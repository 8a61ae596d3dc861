// fp32 FMA GEMM for shapes the tensor-core kernel does not take (tiny or unaligned dimensions, e.g. the
// 10-class output layer).  128x128x8 block tile, 8x8 register tile per thread, any of the four operand
// layouts through (row, k) strides, fused bias / activation / pre-activation epilogue.
#include "common.cuh"

namespace {

constexpr int BM = 128, BN = 128, BK = 8, TM = 8, TN = 8, THREADS = 256;

__global__ void __launch_bounds__(THREADS)
gemm_simt_kernel(const float* __restrict__ A, int64_t a_sm, int64_t a_sk, const float* __restrict__ B, int64_t b_sn,
                 int64_t b_sk, float* __restrict__ C, int64_t ldc, float* __restrict__ Z,
                 const float* __restrict__ bias_n, const float* __restrict__ bias_m, int64_t M, int64_t N, int64_t K,
                 int act, int accumulate) {
  __shared__ float As[2][BK][BM + 4];
  __shared__ float Bs[2][BK][BN + 4];
  const int tid = threadIdx.x;
  const int64_t m0 = (int64_t)blockIdx.y * BM, n0 = (int64_t)blockIdx.x * BN;
  const int tr = tid / 16, tc = tid % 16;  // 16 x 16 thread grid, each 8 x 8 outputs (strided by 16)

  // load mapping: element e = tid + i*256 of the 128 x 8 tile; fastest index follows the unit stride
  const bool a_k_fast = (a_sk == 1), b_k_fast = (b_sk == 1);
  float acc[TM][TN];
#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int j = 0; j < TN; ++j) acc[i][j] = 0.0f;

  float ra[4], rb[4];
  auto load_tiles = [&](int64_t k0) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int e = tid + i * THREADS;
      const int mm = a_k_fast ? e / BK : e % BM, kk = a_k_fast ? e % BK : e / BM;
      const int64_t gm = m0 + mm, gk = k0 + kk;
      ra[i] = (gm < M && gk < K) ? __ldg(A + gm * a_sm + gk * a_sk) : 0.0f;
      const int nn = b_k_fast ? e / BK : e % BN, kb = b_k_fast ? e % BK : e / BN;
      const int64_t gn = n0 + nn, gkb = k0 + kb;
      rb[i] = (gn < N && gkb < K) ? __ldg(B + gn * b_sn + gkb * b_sk) : 0.0f;
    }
  };
  auto store_tiles = [&](int buf) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int e = tid + i * THREADS;
      const int mm = a_k_fast ? e / BK : e % BM, kk = a_k_fast ? e % BK : e / BM;
      As[buf][kk][mm] = ra[i];
      const int nn = b_k_fast ? e / BK : e % BN, kb = b_k_fast ? e % BK : e / BN;
      Bs[buf][kb][nn] = rb[i];
    }
  };

  const int64_t ktiles = (K + BK - 1) / BK;
  if (ktiles > 0) {
    load_tiles(0);
    store_tiles(0);
  }
  __syncthreads();
  for (int64_t kt = 0; kt < ktiles; ++kt) {
    const int buf = (int)(kt & 1);
    if (kt + 1 < ktiles) load_tiles((kt + 1) * BK);
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      float a[TM], b[TN];
#pragma unroll
      for (int i = 0; i < TM; ++i) a[i] = As[buf][kk][tr + 16 * i];
#pragma unroll
      for (int j = 0; j < TN; ++j) b[j] = Bs[buf][kk][tc + 16 * j];
#pragma unroll
      for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    if (kt + 1 < ktiles) store_tiles(buf ^ 1);
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < TM; ++i) {
    const int64_t gm = m0 + tr + 16 * i;
    if (gm >= M) continue;
#pragma unroll
    for (int j = 0; j < TN; ++j) {
      const int64_t gn = n0 + tc + 16 * j;
      if (gn >= N) continue;
      float v = acc[i][j];
      if (accumulate) v += C[gm * ldc + gn];
      if (bias_n) v += __ldg(bias_n + gn);
      if (bias_m) v += __ldg(bias_m + gm);
      if (Z) Z[gm * ldc + gn] = v;
      C[gm * ldc + gn] = fb_act_apply(act, v);
    }
  }
}

}  // namespace

int32_t fb_gemm_simt_launch(fb_ctx* ctx, cudaStream_t stream, const fb_gemm_args& a) {
  (void)ctx;
  if (a.M == 0 || a.N == 0) return FB_OK;
  const int64_t a_sm = a.a_mn_major ? 1 : a.lda, a_sk = a.a_mn_major ? a.lda : 1;
  const int64_t b_sn = a.b_mn_major ? 1 : a.ldb, b_sk = a.b_mn_major ? a.ldb : 1;
  const int64_t gx = (a.N + BN - 1) / BN, gy = (a.M + BM - 1) / BM;
  FB_REQUIRE(gy <= 65535, FB_ERR_SHAPE, "gemm: M = %lld is too large for the FMA kernel", (long long)a.M);
  dim3 grid((unsigned)gx, (unsigned)gy);
  gemm_simt_kernel<<<grid, THREADS, 0, stream>>>(a.A, a_sm, a_sk, a.B, b_sn, b_sk, a.C, a.ldc, a.Z, a.bias_n, a.bias_m,
                                                 a.M, a.N, a.K, a.act, a.accumulate);
  FB_LAUNCH_CHECK();
  return FB_OK;
}
