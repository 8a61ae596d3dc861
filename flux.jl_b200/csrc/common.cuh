// Shared declarations of libfluxb200: context, error reporting, launch helpers, activations.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>

#include "../../include/fluxb200.h"

#define FB_API extern "C" __attribute__((visibility("default")))

// ---------------------------------------------------------------------------- context ---
constexpr int FB_MAX_RETIRED = 64;   // the arena doubles, so this is never reached

struct fb_ctx {
  int device;
  int sm_count;
  int reserved_sms;      // SMs the persistent GEMM leaves free (for communication kernels running beside it)
  size_t smem_optin;
  void* scratch;         // device arena, grown on demand, reused by every call on this context
  size_t scratch_bytes;
  void* retired[FB_MAX_RETIRED];   // outgrown arena blocks, released with the context
  int retired_count;
  int32_t* dev_error;    // device error word written by kernels whose bounded waits ran out
  void* gemm_ws;      // opaque (gemm_tc.cu): workspace of the split-tile GEMM schedule
};

// thread-local last-error message
void fb_set_error(const char* fmt, ...);
int32_t fb_fail(int32_t code, const char* fmt, ...);

// Returns a pointer into the context arena of at least `bytes` (256-byte aligned); grows the arena when it is
// too small (outgrown blocks are kept until fb_ctx_destroy).  NULL on allocation failure.
void* fb_scratch(fb_ctx* ctx, cudaStream_t stream, size_t bytes);

#define FB_CHECK_CTX(ctx)                                                   \
  do {                                                                      \
    if ((ctx) == nullptr) return fb_fail(FB_ERR_INVALID_ARG, "%s: ctx is NULL", __func__); \
  } while (0)

#define FB_CUDA(call)                                                                        \
  do {                                                                                       \
    cudaError_t e__ = (call);                                                                \
    if (e__ != cudaSuccess)                                                                  \
      return fb_fail(FB_ERR_CUDA, "%s: %s failed: %s", __func__, #call, cudaGetErrorString(e__)); \
  } while (0)

extern unsigned long long g_fb_kernel_launches;   // kernels launched by this library in this process

#define FB_LAUNCH_CHECK()                                                                     \
  do {                                                                                        \
    ++g_fb_kernel_launches;                                                                   \
    cudaError_t e__ = cudaGetLastError();                                                     \
    if (e__ != cudaSuccess)                                                                   \
      return fb_fail(FB_ERR_CUDA, "%s: kernel launch failed: %s", __func__, cudaGetErrorString(e__)); \
  } while (0)

#define FB_REQUIRE(cond, code, ...)                    \
  do {                                                 \
    if (!(cond)) return fb_fail((code), __VA_ARGS__);  \
  } while (0)

static inline bool fb_aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// ------------------------------------------------------------------------ activations ---
// Evaluated in fp32.  *_from_y derivatives use the forward output where that is enough
// (relu / tanh / sigmoid), the gelu flavours need the pre-activation z.
__device__ __forceinline__ float fb_sigmoidf(float z) { return 1.0f / (1.0f + __expf(-z)); }

__device__ __forceinline__ float fb_act_apply(int act, float z) {
  switch (act) {
    case FB_ACT_RELU: return fmaxf(z, 0.0f);
    case FB_ACT_TANH: return tanhf(z);
    case FB_ACT_SIGMOID: return 1.0f / (1.0f + expf(-z));
    case FB_ACT_GELU_TANH: {
      const float u = 0.7978845608028654f * (z + 0.044715f * z * z * z);
      return 0.5f * z * (1.0f + tanhf(u));
    }
    case FB_ACT_GELU_ERF: return 0.5f * z * (1.0f + erff(z * 0.7071067811865476f));
    default: return z;
  }
}

// derivative at pre-activation z
__device__ __forceinline__ float fb_act_grad_z(int act, float z) {
  switch (act) {
    case FB_ACT_RELU: return z > 0.0f ? 1.0f : 0.0f;
    case FB_ACT_TANH: { const float t = tanhf(z); return 1.0f - t * t; }
    case FB_ACT_SIGMOID: { const float s = 1.0f / (1.0f + expf(-z)); return s * (1.0f - s); }
    case FB_ACT_GELU_TANH: {
      const float z2 = z * z;
      const float u = 0.7978845608028654f * (z + 0.044715f * z * z2);
      const float t = tanhf(u);
      const float du = 0.7978845608028654f * (1.0f + 3.0f * 0.044715f * z2);
      return 0.5f * (1.0f + t) + 0.5f * z * (1.0f - t * t) * du;
    }
    case FB_ACT_GELU_ERF: {
      const float pdf = 0.3989422804014327f * expf(-0.5f * z * z);
      return 0.5f * (1.0f + erff(z * 0.7071067811865476f)) + z * pdf;
    }
    default: return 1.0f;
  }
}

// derivative from the forward output y (valid for identity / relu / tanh / sigmoid)
__device__ __forceinline__ float fb_act_grad_y(int act, float y) {
  switch (act) {
    case FB_ACT_RELU: return y > 0.0f ? 1.0f : 0.0f;
    case FB_ACT_TANH: return 1.0f - y * y;
    case FB_ACT_SIGMOID: return y * (1.0f - y);
    default: return 1.0f;
  }
}

static inline bool fb_act_valid(int act) { return act >= FB_ACT_IDENTITY && act <= FB_ACT_GELU_ERF; }
static inline bool fb_act_needs_z(int act) { return act == FB_ACT_GELU_TANH || act == FB_ACT_GELU_ERF; }

// ------------------------------------------------------------------ counter-based random numbers ---
// Philox4x32-10 (Salmon et al., "Parallel random numbers: as easy as 1, 2, 3"), 64-bit counter, 64-bit key.
__device__ __forceinline__ void philox_round(uint32_t (&c)[4], uint32_t k0, uint32_t k1) {
  const uint64_t p0 = (uint64_t)0xD2511F53u * c[0], p1 = (uint64_t)0xCD9E8D57u * c[2];
  const uint32_t n0 = (uint32_t)(p1 >> 32) ^ c[1] ^ k0, n1 = (uint32_t)p1;
  const uint32_t n2 = (uint32_t)(p0 >> 32) ^ c[3] ^ k1, n3 = (uint32_t)p0;
  c[0] = n0; c[1] = n1; c[2] = n2; c[3] = n3;
}
__device__ __forceinline__ void philox4x32_10(uint64_t counter, uint64_t seed, uint32_t (&out)[4]) {
  uint32_t c[4] = {(uint32_t)counter, (uint32_t)(counter >> 32), 0u, 0u};
  uint32_t k0 = (uint32_t)seed, k1 = (uint32_t)(seed >> 32);
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    philox_round(c, k0, k1);
    k0 += 0x9E3779B9u;
    k1 += 0xBB67AE85u;
  }
  out[0] = c[0]; out[1] = c[1]; out[2] = c[2]; out[3] = c[3];
}

// Dropout keep decision for element `idx` of a mask stream: word idx % 4 of Philox(counter = offset + idx / 4).
__device__ __forceinline__ bool fb_dropout_keep(uint64_t idx, float p, uint64_t seed, uint64_t offset) {
  uint32_t r[4];
  philox4x32_10((idx >> 2) + offset, seed, r);
  const uint32_t w = (idx & 3) == 0 ? r[0] : (idx & 3) == 1 ? r[1] : (idx & 3) == 2 ? r[2] : r[3];
  return (float)(w >> 8) * (1.0f / 16777216.0f) >= p;
}

// -------------------------------------------------------------------------- reductions ---
__device__ __forceinline__ float fb_warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float fb_warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Block-wide sum; `sh` must hold at least 32 floats.  All threads get the result.
__device__ __forceinline__ float fb_block_sum(float v, float* sh) {
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = fb_warp_sum(v);
  __syncthreads();
  if (lane == 0) sh[w] = v;
  __syncthreads();
  float r = (lane < nw) ? sh[lane] : 0.0f;
  r = fb_warp_sum(r);
  return r;
}
__device__ __forceinline__ float fb_block_max(float v, float* sh) {
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = fb_warp_max(v);
  __syncthreads();
  if (lane == 0) sh[w] = v;
  __syncthreads();
  float r = (lane < nw) ? sh[lane] : -INFINITY;
  r = fb_warp_max(r);
  return r;
}

// Welford / Chan merge of (count, mean, M2) partials
__device__ __forceinline__ void fb_welford_merge(float& n_a, float& mean_a, float& m2_a, float n_b,
                                                 float mean_b, float m2_b) {
  if (n_b == 0.0f) return;
  const float n = n_a + n_b;
  const float delta = mean_b - mean_a;
  const float f = n_b / n;
  mean_a += delta * f;
  m2_a += m2_b + delta * delta * n_a * f;
  n_a = n;
}

// ---------------------------------------------------------- internal cross-file entry points ---
// Row-major core GEMM: C[M][N] (ldc) = A*B with A given either K-major (A[m*lda + k]) or MN-major
// (A[k*lda + m]), same for B (K-major: B[n*ldb + k]; MN-major: B[k*ldb + n]).  Epilogue: optional bias
// along n, activation, optional pre-activation store, optional accumulate into C.
struct fb_gemm_args {
  const float* A; int64_t lda; int a_mn_major;
  const float* B; int64_t ldb; int b_mn_major;
  float* C; int64_t ldc;
  float* Z;              // optional pre-activation (same layout as C), or NULL
  const float* bias_n;   // optional bias indexed by n, or NULL
  const float* bias_m;   // optional bias indexed by m, or NULL
  int64_t M, N, K;
  int act;
  int accumulate;
};
// bf16 operands (raw uint16 bit patterns), fp32 accumulation; C is bf16 (or fp32 when out_f32), Z / bias_n are bf16
struct fb_gemm_bf16_args {
  const uint16_t* A; int64_t lda; int a_mn_major;
  const uint16_t* B; int64_t ldb; int b_mn_major;
  void* C; int64_t ldc;
  uint16_t* Z;
  const uint16_t* bias_n;
  int64_t M, N, K;
  int act;
  int accumulate;
  int out_f32;
};
int32_t fb_gemm_bf16_launch(fb_ctx* ctx, cudaStream_t stream, const fb_gemm_bf16_args& a);
bool fb_gemm_bf16_supported(const fb_gemm_bf16_args& a);
int32_t fb_gemm_simt_launch(fb_ctx* ctx, cudaStream_t stream, const fb_gemm_args& a);
// tensor-core path; returns FB_ERR_UNSUPPORTED (without raising an error message) when the shape or
// alignment is outside what the kernel handles, so the dispatcher can pick the FMA kernel.
int32_t fb_gemm_tc_launch(fb_ctx* ctx, cudaStream_t stream, const fb_gemm_args& a, int passes);
bool fb_gemm_tc_supported(const fb_gemm_args& a);
int32_t fb_gemm_dispatch(fb_ctx* ctx, cudaStream_t stream, const fb_gemm_args& a, int precision);
void fb_gemm_workspace_destroy(fb_ctx* ctx);
// attention_tc.cu: tensor-core attention forward; FB_ERR_UNSUPPORTED when the shape is not taken
int32_t fb_attn_fwd_tc(fb_ctx* ctx, cudaStream_t stream, const float* q, const float* k, const float* v, const uint8_t* mask,
                       float* o, float* lse, int64_t e_dim, int64_t ev_dim, int64_t lq, int64_t lk, int64_t batch, int nheads,
                       int causal);
int32_t fb_attn_bwd_dq_tc(fb_ctx* ctx, cudaStream_t stream, const float* q, const float* k, const float* v, const uint8_t* mask,
                          const float* lse, const float* dlt, const float* dout, float* dq, int64_t e_dim, int64_t ev_dim,
                          int64_t lq, int64_t lk, int64_t batch, int nheads, int causal);
int32_t fb_attn_bwd_dkdv_tc(fb_ctx* ctx, cudaStream_t stream, const float* q, const float* k, const float* v, const uint8_t* mask,
                            const float* lse, const float* dlt, const float* dout, float* dk, float* dv, int64_t e_dim,
                            int64_t ev_dim, int64_t lq, int64_t lk, int64_t batch, int nheads, int causal);
int32_t fb_gemm_workspace_create(fb_ctx* ctx);
// Kernels that run on a communication stream beside a resident GEMM CTA (update, peer exchange, time marks) ask for
// the same shared-memory carve-out as the GEMM: an SM runs CTAs of different kernels together only when they agree
// on how its L1 / shared memory is split.
int32_t fb_side_kernels_prepare_elementwise();
int32_t fb_side_kernels_prepare_peer();
void fb_gemm_workspace_reset(fb_ctx* ctx, cudaStream_t stream);

// delta = dy .* act'(.) and db[j] = sum_rows delta[row][j]   (rows x cols row-major; cols = out_dim)
int32_t fb_act_bwd_colsum(fb_ctx* ctx, cudaStream_t stream, int act, const float* dy, const float* y,
                          const float* z, float* delta, float* db, int64_t rows, int64_t cols);
