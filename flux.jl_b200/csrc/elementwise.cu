// Element-wise helpers, the loss kernels and the multi-tensor Adam step (all memory-bound).
#include "common.cuh"

namespace {

constexpr int EW_THREADS = 256;

unsigned ew_grid(const fb_ctx* ctx, int64_t items) {
  int64_t blocks = (items + EW_THREADS - 1) / EW_THREADS;
  const int64_t cap = (int64_t)ctx->sm_count * 32;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  return (unsigned)blocks;
}

__global__ void __launch_bounds__(EW_THREADS)
scale_kernel(const float* __restrict__ x, float alpha, float* __restrict__ y, int64_t count, int vec) {
  const int64_t tid = (int64_t)blockIdx.x * EW_THREADS + threadIdx.x, stride = (int64_t)gridDim.x * EW_THREADS;
  if (vec) {
    const float4* x4 = (const float4*)x;
    float4* y4 = (float4*)y;
    for (int64_t i = tid; i < (count >> 2); i += stride) {
      float4 v = __ldcs(x4 + i);
      v.x *= alpha; v.y *= alpha; v.z *= alpha; v.w *= alpha;
      __stcs(y4 + i, v);
    }
    for (int64_t i = (count & ~int64_t(3)) + tid; i < count; i += stride) y[i] = alpha * x[i];
  } else {
    for (int64_t i = tid; i < count; i += stride) y[i] = alpha * x[i];
  }
}

__global__ void __launch_bounds__(EW_THREADS)
axpy_kernel(float alpha, const float* __restrict__ x, float* __restrict__ y, int64_t count, int vec) {
  const int64_t tid = (int64_t)blockIdx.x * EW_THREADS + threadIdx.x, stride = (int64_t)gridDim.x * EW_THREADS;
  if (vec) {
    const float4* x4 = (const float4*)x;
    float4* y4 = (float4*)y;
    for (int64_t i = tid; i < (count >> 2); i += stride) {
      const float4 a = __ldcs(x4 + i);
      float4 b = y4[i];
      b.x = fmaf(alpha, a.x, b.x); b.y = fmaf(alpha, a.y, b.y); b.z = fmaf(alpha, a.z, b.z); b.w = fmaf(alpha, a.w, b.w);
      y4[i] = b;
    }
    for (int64_t i = (count & ~int64_t(3)) + tid; i < count; i += stride) y[i] = fmaf(alpha, x[i], y[i]);
  } else {
    for (int64_t i = tid; i < count; i += stride) y[i] = fmaf(alpha, x[i], y[i]);
  }
}

// bf16 bits by round-to-nearest-even in the integer domain, NaN -> 0x7fc0
__device__ __forceinline__ uint16_t f32_to_bf16_bits(float f) {
  const uint32_t u = __float_as_uint(f);
  const uint32_t r = (u + 0x00007fffu + ((u >> 16) & 1u)) >> 16;
  return (f != f) ? (uint16_t)0x7fc0 : (uint16_t)r;
}

__global__ void __launch_bounds__(EW_THREADS)
cast_f32_bf16_kernel(const float* __restrict__ x, uint16_t* __restrict__ y, int64_t count) {
  const int64_t tid = (int64_t)blockIdx.x * EW_THREADS + threadIdx.x, stride = (int64_t)gridDim.x * EW_THREADS;
  for (int64_t i = tid; i < count; i += stride) y[i] = f32_to_bf16_bits(x[i]);
}

__global__ void __launch_bounds__(EW_THREADS)
cast_bf16_f32_kernel(const uint16_t* __restrict__ x, float* __restrict__ y, int64_t count) {
  const int64_t tid = (int64_t)blockIdx.x * EW_THREADS + threadIdx.x, stride = (int64_t)gridDim.x * EW_THREADS;
  for (int64_t i = tid; i < count; i += stride) y[i] = __uint_as_float((uint32_t)x[i] << 16);
}

// ------------------------------------------------------------------------------- sum of squares ---
__global__ void __launch_bounds__(EW_THREADS)
sumsq_partial_kernel(const float* __restrict__ x, int64_t count, float* __restrict__ part, int vec, int square) {
  __shared__ float sh[32];
  const int64_t tid = (int64_t)blockIdx.x * EW_THREADS + threadIdx.x, stride = (int64_t)gridDim.x * EW_THREADS;
  float s = 0.0f;
  if (vec) {
    const float4* x4 = (const float4*)x;
    for (int64_t i = tid; i < (count >> 2); i += stride) {
      const float4 v = __ldcs(x4 + i);
      s += square ? (v.x * v.x + v.y * v.y) + (v.z * v.z + v.w * v.w) : (v.x + v.y) + (v.z + v.w);
    }
    for (int64_t i = (count & ~int64_t(3)) + tid; i < count; i += stride) s += square ? x[i] * x[i] : x[i];
  } else {
    for (int64_t i = tid; i < count; i += stride) s += square ? x[i] * x[i] : x[i];
  }
  s = fb_block_sum(s, sh);
  if (threadIdx.x == 0) part[blockIdx.x] = s;
}

// out[0] = scale * sum(part[0..m))   (one block; fixed order -> run-to-run deterministic)
__global__ void __launch_bounds__(1024)
final_sum_kernel(const float* __restrict__ part, int64_t m, float scale, float* __restrict__ out) {
  __shared__ float sh[32];
  float s = 0.0f;
  for (int64_t i = threadIdx.x; i < m; i += 1024) s += part[i];
  s = fb_block_sum(s, sh);
  if (threadIdx.x == 0) out[0] = s * scale;
}

// ------------------------------------------------------------------------ logit cross-entropy ---
// One warp per sample (column of Julia yhat[c, n] = row of the [n][c] buffer).
template <bool LABELS>
__global__ void __launch_bounds__(128)
xent_kernel(const float* __restrict__ yhat, const int32_t* __restrict__ labels, const float* __restrict__ ydense,
            float* __restrict__ loss_part, float* __restrict__ dyhat, int64_t c, int64_t n, float gscale) {
  const int lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * 4 + (threadIdx.x >> 5);
  if (row >= n) return;
  const float* z = yhat + row * c;
  float mx = -INFINITY;
  for (int64_t j = lane; j < c; j += 32) mx = fmaxf(mx, z[j]);
  mx = fb_warp_max(mx);
  float se = 0.0f, sy = 0.0f, syz = 0.0f;
  for (int64_t j = lane; j < c; j += 32) {
    const float zj = z[j];
    se += expf(zj - mx);
    if (!LABELS) {
      const float yj = ydense[row * c + j];
      sy += yj;
      syz += yj * zj;
    }
  }
  se = fb_warp_sum(se);
  const float lse = mx + logf(se);
  int64_t lab = 0;
  if (LABELS) {
    lab = (int64_t)labels[row] - 1;  // labels are 1-based, as onehotbatch(labels, 1:c)
    sy = 1.0f;
    syz = (lab >= 0 && lab < c) ? z[lab] : 0.0f;
  } else {
    sy = fb_warp_sum(sy);
    syz = fb_warp_sum(syz);
  }
  // -sum_j y_j (z_j - lse) = lse * sum(y) - sum(y z)
  if (lane == 0) loss_part[row] = lse * sy - syz;
  if (dyhat != nullptr) {
    float* d = dyhat + row * c;
    for (int64_t j = lane; j < c; j += 32) {
      const float p = expf(z[j] - lse);
      const float yj = LABELS ? (j == lab ? 1.0f : 0.0f) : ydense[row * c + j];
      d[j] = (p * sy - yj) * gscale;
    }
  }
}

// ------------------------------------------------------------------------------------- Adam ---
constexpr int ADAM_MAX_TENSORS = 32;
constexpr int ADAM_CHUNK = 8192;  // elements per block

struct AdamTable {
  float* w[ADAM_MAX_TENSORS];
  const float* g[ADAM_MAX_TENSORS];
  float* m[ADAM_MAX_TENSORS];
  float* v[ADAM_MAX_TENSORS];
  long long count[ADAM_MAX_TENSORS];
  int block_start[ADAM_MAX_TENSORS + 1];
  int ntensors;
};

// Two shapes of one kernel.  The plain one (256 threads) streams at the HBM roofline when it has the GPU to itself.
// The side one (128 threads of at most 32 registers) fits on an SM beside a resident GEMM CTA - one warp per
// register-file partition - so an update enqueued on the communication stream does not wait for the reverse sweep's
// GEMM to end; alone it reaches about 70 % of the plain one's bandwidth.
constexpr int ADAM_SIDE_THREADS = 128;
template <int ADAM_THREADS, int MIN_BLOCKS>
__global__ void __launch_bounds__(ADAM_THREADS, MIN_BLOCKS)
adam_kernel(const __grid_constant__ AdamTable tab, float eta, float beta1, float beta2, float eps, float inv_c1,
            float inv_c2, float grad_scale, const float* __restrict__ bt_dev, const float* __restrict__ guard) {
  // device-resident step state (used when the step is replayed from a CUDA graph): the running beta powers
  // and an optional guard scalar (the loss) whose non-finite value skips the update
  if (guard != nullptr && !isfinite(__ldg(guard))) return;
  if (bt_dev != nullptr) {
    inv_c1 = 1.0f / (1.0f - __ldg(bt_dev));
    inv_c2 = 1.0f / (1.0f - __ldg(bt_dev + 1));
  }
  int t = 0;
  while (t + 1 < tab.ntensors && (int)blockIdx.x >= tab.block_start[t + 1]) ++t;
  const int64_t begin = (int64_t)(blockIdx.x - tab.block_start[t]) * ADAM_CHUNK;
  const int64_t count = tab.count[t];
  int64_t end = begin + ADAM_CHUNK;
  if (end > count) end = count;
  float* w = tab.w[t];
  const float* g = tab.g[t];
  float* m = tab.m[t];
  float* v = tab.v[t];
  const float omb1 = 1.0f - beta1, omb2 = 1.0f - beta2;
  const bool vec = ((reinterpret_cast<uintptr_t>(w) | reinterpret_cast<uintptr_t>(g) | reinterpret_cast<uintptr_t>(m) |
                     reinterpret_cast<uintptr_t>(v)) & 15u) == 0;
  if (vec) {
    const int64_t e4 = begin + ((end - begin) & ~int64_t(3));
    for (int64_t i = begin + 4 * threadIdx.x; i < e4; i += 4 * ADAM_THREADS) {
      float4 gv = __ldcs((const float4*)(g + i));
      float4 mv = *(const float4*)(m + i), vv = *(const float4*)(v + i), wv = *(const float4*)(w + i);
      float* gp = &gv.x; float* mp = &mv.x; float* vp = &vv.x; float* wp = &wv.x;
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float gk = gp[k] * grad_scale;
        mp[k] = beta1 * mp[k] + omb1 * gk;
        vp[k] = beta2 * vp[k] + omb2 * gk * gk;
        wp[k] -= mp[k] * inv_c1 / (sqrtf(vp[k] * inv_c2) + eps) * eta;
      }
      *(float4*)(m + i) = mv;
      *(float4*)(v + i) = vv;
      *(float4*)(w + i) = wv;
    }
    for (int64_t i = e4 + threadIdx.x; i < end; i += ADAM_THREADS) {
      const float gk = g[i] * grad_scale;
      const float mk = beta1 * m[i] + omb1 * gk, vk = beta2 * v[i] + omb2 * gk * gk;
      m[i] = mk; v[i] = vk;
      w[i] -= mk * inv_c1 / (sqrtf(vk * inv_c2) + eps) * eta;
    }
  } else {
    for (int64_t i = begin + threadIdx.x; i < end; i += ADAM_THREADS) {
      const float gk = g[i] * grad_scale;
      const float mk = beta1 * m[i] + omb1 * gk, vk = beta2 * v[i] + omb2 * gk * gk;
      m[i] = mk; v[i] = vk;
      w[i] -= mk * inv_c1 / (sqrtf(vk * inv_c2) + eps) * eta;
    }
  }
}

// ------------------------------------------------- activation backward + bias-gradient column sum ---
// delta[r][j] = dy[r][j] * act'(.) ; part[blockIdx.y][j] = sum over this block's rows of delta[r][j].
// Block = 32 x 8 threads; thread (tx, ty) owns VEC consecutive columns.
template <int VEC>
__global__ void __launch_bounds__(256)
act_bwd_colsum_kernel(int act, const float* __restrict__ dy, const float* __restrict__ y, const float* __restrict__ z,
                      float* __restrict__ delta, float* __restrict__ part, int64_t rows, int64_t cols,
                      int64_t rows_per_block) {
  __shared__ float sh[8][32 * VEC + 1];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const int64_t col0 = ((int64_t)blockIdx.x * 32 + tx) * VEC;
  const int64_t r_begin = (int64_t)blockIdx.y * rows_per_block;
  int64_t r_end = r_begin + rows_per_block;
  if (r_end > rows) r_end = rows;
  float acc[VEC];
#pragma unroll
  for (int k = 0; k < VEC; ++k) acc[k] = 0.0f;
  if (col0 < cols) {
    for (int64_t r = r_begin + ty; r < r_end; r += 8) {
      const int64_t off = r * cols + col0;
      float d[VEC];
      if (VEC == 4) {
        const float4 dv = __ldcs((const float4*)(dy + off));
        d[0] = dv.x; d[1] = dv.y; d[2] = dv.z; d[3] = dv.w;
        if (act != FB_ACT_IDENTITY) {
          const bool use_z = (act == FB_ACT_GELU_TANH || act == FB_ACT_GELU_ERF);
          const float4 sv = __ldcs((const float4*)((use_z ? z : y) + off));
          const float s[4] = {sv.x, sv.y, sv.z, sv.w};
#pragma unroll
          for (int k = 0; k < 4; ++k) d[k] *= use_z ? fb_act_grad_z(act, s[k]) : fb_act_grad_y(act, s[k]);
        }
        if (delta != nullptr) __stcs((float4*)(delta + off), make_float4(d[0], d[1], d[2], d[3]));
      } else {
        d[0] = dy[off];
        if (act != FB_ACT_IDENTITY) {
          const bool use_z = (act == FB_ACT_GELU_TANH || act == FB_ACT_GELU_ERF);
          d[0] *= use_z ? fb_act_grad_z(act, z[off]) : fb_act_grad_y(act, y[off]);
        }
        if (delta != nullptr) delta[off] = d[0];
      }
#pragma unroll
      for (int k = 0; k < VEC; ++k) acc[k] += d[k];
    }
  }
  if (part == nullptr) return;
#pragma unroll
  for (int k = 0; k < VEC; ++k) sh[ty][tx * VEC + k] = acc[k];
  __syncthreads();
  if (ty == 0 && col0 < cols) {
#pragma unroll
    for (int k = 0; k < VEC; ++k) {
      float s = 0.0f;
#pragma unroll
      for (int i = 0; i < 8; ++i) s += sh[i][tx * VEC + k];
      part[(int64_t)blockIdx.y * cols + col0 + k] = s;
    }
  }
}

}  // namespace

__global__ void fb_colreduce2_kernel(const float* part_a, const float* part_b, float* out_a, float* out_b,
                                     int64_t groups, int64_t d);

int32_t fb_act_bwd_colsum(fb_ctx* ctx, cudaStream_t stream, int act, const float* dy, const float* y,
                          const float* z, float* delta, float* db, int64_t rows, int64_t cols) {
  const bool need_delta = (act != FB_ACT_IDENTITY);
  if (!need_delta && db == nullptr) return FB_OK;
  if (need_delta) {
    FB_REQUIRE(delta != nullptr, FB_ERR_INVALID_ARG, "dense backward: delta scratch is required for a non-identity activation");
    if (fb_act_needs_z(act)) FB_REQUIRE(z != nullptr, FB_ERR_INVALID_ARG, "dense backward: the gelu activations need the saved pre-activation z");
    else FB_REQUIRE(y != nullptr, FB_ERR_INVALID_ARG, "dense backward: the forward output y is required");
  }
  const float* src = fb_act_needs_z(act) ? z : y;
  const bool vec = (cols % 4 == 0) && fb_aligned16(dy) && (!need_delta || (fb_aligned16(delta) && fb_aligned16(src)));
  const int V = vec ? 4 : 1;
  const int64_t gx = (cols + 32 * V - 1) / (32 * V);
  int64_t gy = ((int64_t)ctx->sm_count * 8 + gx - 1) / gx;
  if (gy > (rows + 7) / 8) gy = (rows + 7) / 8;
  if (gy < 1) gy = 1;
  if (gy > 65535) gy = 65535;
  const int64_t rpb = (rows + gy - 1) / gy;
  gy = (rows + rpb - 1) / rpb;
  float* part = nullptr;
  if (db != nullptr) {
    part = (float*)fb_scratch(ctx, stream, (size_t)(gy * cols) * sizeof(float));
    if (!part) return FB_ERR_ALLOC;
  }
  dim3 grid((unsigned)gx, (unsigned)gy);
  float* dout = need_delta ? delta : nullptr;
  if (vec) act_bwd_colsum_kernel<4><<<grid, 256, 0, stream>>>(act, dy, y, z, dout, part, rows, cols, rpb);
  else act_bwd_colsum_kernel<1><<<grid, 256, 0, stream>>>(act, dy, y, z, dout, part, rows, cols, rpb);
  FB_LAUNCH_CHECK();
  if (db != nullptr) {
    fb_colreduce2_kernel<<<(unsigned)((cols + 31) / 32), 256, 0, stream>>>(part, nullptr, db, nullptr, gy, cols);
    FB_LAUNCH_CHECK();
  }
  return FB_OK;
}

FB_API int32_t fb_scale(fb_ctx* ctx, void* stream, const float* x, float alpha, float* y, int64_t count) {
  FB_CHECK_CTX(ctx);
  FB_REQUIRE(count >= 0, FB_ERR_INVALID_ARG, "fb_scale: negative count");
  if (count == 0) return FB_OK;
  FB_REQUIRE(x && y, FB_ERR_INVALID_ARG, "fb_scale: NULL pointer");
  const int vec = fb_aligned16(x) && fb_aligned16(y);
  scale_kernel<<<ew_grid(ctx, vec ? (count + 3) / 4 : count), EW_THREADS, 0, (cudaStream_t)stream>>>(x, alpha, y, count, vec);
  FB_LAUNCH_CHECK();
  return FB_OK;
}

__global__ void __launch_bounds__(256) fill_kernel(float* __restrict__ x, float value, int64_t count) {
  for (int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x; i < count; i += (int64_t)gridDim.x * 256) x[i] = value;
}

FB_API int32_t fb_fill(fb_ctx* ctx, void* stream, float* x, float value, int64_t count) {
  FB_CHECK_CTX(ctx);
  FB_REQUIRE(count >= 0, FB_ERR_INVALID_ARG, "fb_fill: negative count");
  if (count == 0) return FB_OK;
  FB_REQUIRE(x, FB_ERR_INVALID_ARG, "fb_fill: NULL pointer");
  int64_t blocks = (count + 255) / 256;
  if (blocks > (int64_t)ctx->sm_count * 32) blocks = (int64_t)ctx->sm_count * 32;
  fill_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(x, value, count);
  FB_LAUNCH_CHECK();
  return FB_OK;
}

// One thread stores the GPU's nanosecond timer: a stream-ordered time mark that also works inside a captured graph
// (where events cannot be timed).
__global__ void timestamp_kernel(uint64_t* out) {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  *out = t;
}

int32_t fb_side_kernels_prepare_elementwise() {
  FB_CUDA(cudaFuncSetAttribute(adam_kernel<ADAM_SIDE_THREADS, 2048 / ADAM_SIDE_THREADS>, cudaFuncAttributePreferredSharedMemoryCarveout,
                               cudaSharedmemCarveoutMaxShared));
  FB_CUDA(cudaFuncSetAttribute(timestamp_kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared));
  return FB_OK;
}

FB_API int32_t fb_timestamp(fb_ctx* ctx, void* stream, uint64_t* out_dev) {
  FB_CHECK_CTX(ctx);
  FB_REQUIRE(out_dev, FB_ERR_INVALID_ARG, "fb_timestamp: NULL pointer");
  timestamp_kernel<<<1, 1, 0, (cudaStream_t)stream>>>(out_dev);
  FB_LAUNCH_CHECK();
  return FB_OK;
}

FB_API int32_t fb_axpy(fb_ctx* ctx, void* stream, float alpha, const float* x, float* y, int64_t count) {
  FB_CHECK_CTX(ctx);
  FB_REQUIRE(count >= 0, FB_ERR_INVALID_ARG, "fb_axpy: negative count");
  if (count == 0) return FB_OK;
  FB_REQUIRE(x && y, FB_ERR_INVALID_ARG, "fb_axpy: NULL pointer");
  const int vec = fb_aligned16(x) && fb_aligned16(y);
  axpy_kernel<<<ew_grid(ctx, vec ? (count + 3) / 4 : count), EW_THREADS, 0, (cudaStream_t)stream>>>(alpha, x, y, count, vec);
  FB_LAUNCH_CHECK();
  return FB_OK;
}

__global__ void __launch_bounds__(EW_THREADS)
round_bf16_kernel(const float* __restrict__ x, float* __restrict__ y, int64_t count) {
  const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x, stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = tid; i < count; i += stride) y[i] = __uint_as_float((uint32_t)f32_to_bf16_bits(x[i]) << 16);
}

FB_API int32_t fb_round_bf16(fb_ctx* ctx, void* stream, const float* x, float* y, int64_t count) {
  FB_CHECK_CTX(ctx);
  FB_REQUIRE(count >= 0, FB_ERR_INVALID_ARG, "fb_round_bf16: negative count");
  if (count == 0) return FB_OK;
  FB_REQUIRE(x && y, FB_ERR_INVALID_ARG, "fb_round_bf16: NULL pointer");
  round_bf16_kernel<<<ew_grid(ctx, count), EW_THREADS, 0, (cudaStream_t)stream>>>(x, y, count);
  FB_LAUNCH_CHECK();
  return FB_OK;
}

FB_API int32_t fb_cast_f32_bf16(fb_ctx* ctx, void* stream, const float* x, uint16_t* y, int64_t count) {
  FB_CHECK_CTX(ctx);
  FB_REQUIRE(count >= 0, FB_ERR_INVALID_ARG, "fb_cast_f32_bf16: negative count");
  if (count == 0) return FB_OK;
  FB_REQUIRE(x && y, FB_ERR_INVALID_ARG, "fb_cast_f32_bf16: NULL pointer");
  cast_f32_bf16_kernel<<<ew_grid(ctx, count), EW_THREADS, 0, (cudaStream_t)stream>>>(x, y, count);
  FB_LAUNCH_CHECK();
  return FB_OK;
}

FB_API int32_t fb_cast_bf16_f32(fb_ctx* ctx, void* stream, const uint16_t* x, float* y, int64_t count) {
  FB_CHECK_CTX(ctx);
  FB_REQUIRE(count >= 0, FB_ERR_INVALID_ARG, "fb_cast_bf16_f32: negative count");
  if (count == 0) return FB_OK;
  FB_REQUIRE(x && y, FB_ERR_INVALID_ARG, "fb_cast_bf16_f32: NULL pointer");
  cast_bf16_f32_kernel<<<ew_grid(ctx, count), EW_THREADS, 0, (cudaStream_t)stream>>>(x, y, count);
  FB_LAUNCH_CHECK();
  return FB_OK;
}

static int32_t sum_common(fb_ctx* ctx, cudaStream_t stream, const float* x, int64_t count, float* out, int square,
                          const char* fn) {
  FB_REQUIRE(count >= 0 && out, FB_ERR_INVALID_ARG, "%s: bad arguments", fn);
  if (count == 0) {
    FB_CUDA(cudaMemsetAsync(out, 0, sizeof(float), stream));
    return FB_OK;
  }
  FB_REQUIRE(x, FB_ERR_INVALID_ARG, "%s: NULL pointer", fn);
  const int vec = fb_aligned16(x);
  int64_t blocks = ((vec ? count / 4 : count) + EW_THREADS - 1) / EW_THREADS;
  const int64_t cap = (int64_t)ctx->sm_count * 8;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  float* part = (float*)fb_scratch(ctx, stream, (size_t)blocks * sizeof(float));
  if (!part) return FB_ERR_ALLOC;
  sumsq_partial_kernel<<<(unsigned)blocks, EW_THREADS, 0, stream>>>(x, count, part, vec, square);
  FB_LAUNCH_CHECK();
  final_sum_kernel<<<1, 1024, 0, stream>>>(part, blocks, 1.0f, out);
  FB_LAUNCH_CHECK();
  return FB_OK;
}

FB_API int32_t fb_sumsq(fb_ctx* ctx, void* stream, const float* x, int64_t count, float* out) {
  FB_CHECK_CTX(ctx);
  return sum_common(ctx, (cudaStream_t)stream, x, count, out, 1, "fb_sumsq");
}

FB_API int32_t fb_sum(fb_ctx* ctx, void* stream, const float* x, int64_t count, float* out) {
  FB_CHECK_CTX(ctx);
  return sum_common(ctx, (cudaStream_t)stream, x, count, out, 0, "fb_sum");
}

static int32_t xent_common(fb_ctx* ctx, cudaStream_t stream, const float* yhat, const int32_t* labels, const float* y,
                           float* loss, float* dyhat, int64_t c, int64_t n, float dloss, const char* fn) {
  FB_REQUIRE(c >= 1 && n >= 1, FB_ERR_SHAPE, "%s: bad shape c=%lld n=%lld", fn, (long long)c, (long long)n);
  FB_REQUIRE(yhat && loss && (labels || y), FB_ERR_INVALID_ARG, "%s: NULL pointer", fn);
  float* part = (float*)fb_scratch(ctx, stream, (size_t)n * sizeof(float));
  if (!part) return FB_ERR_ALLOC;
  const unsigned grid = (unsigned)((n + 3) / 4);
  const float gscale = dloss / (float)n;
  if (labels) xent_kernel<true><<<grid, 128, 0, stream>>>(yhat, labels, nullptr, part, dyhat, c, n, gscale);
  else xent_kernel<false><<<grid, 128, 0, stream>>>(yhat, nullptr, y, part, dyhat, c, n, gscale);
  FB_LAUNCH_CHECK();
  final_sum_kernel<<<1, 1024, 0, stream>>>(part, n, 1.0f / (float)n, loss);
  FB_LAUNCH_CHECK();
  return FB_OK;
}

FB_API int32_t fb_logitcrossentropy_labels(fb_ctx* ctx, void* stream, const float* yhat, const int32_t* labels,
                                           float* loss, float* dyhat, int64_t c, int64_t n, float dloss) {
  FB_CHECK_CTX(ctx);
  FB_REQUIRE(labels, FB_ERR_INVALID_ARG, "fb_logitcrossentropy_labels: labels is NULL");
  return xent_common(ctx, (cudaStream_t)stream, yhat, labels, nullptr, loss, dyhat, c, n, dloss, "fb_logitcrossentropy_labels");
}

FB_API int32_t fb_logitcrossentropy_dense(fb_ctx* ctx, void* stream, const float* yhat, const float* y, float* loss,
                                          float* dyhat, int64_t c, int64_t n, float dloss) {
  FB_CHECK_CTX(ctx);
  FB_REQUIRE(y, FB_ERR_INVALID_ARG, "fb_logitcrossentropy_dense: y is NULL");
  return xent_common(ctx, (cudaStream_t)stream, yhat, nullptr, y, loss, dyhat, c, n, dloss, "fb_logitcrossentropy_dense");
}

static int32_t adam_common(fb_ctx* ctx, cudaStream_t stream, int32_t ntensors, float* const* w_host,
                           const float* const* g_host, float* const* m_host, float* const* v_host,
                           const int64_t* counts_host, float eta, float beta1, float beta2, float eps, float b1t,
                           float b2t, float grad_scale, const float* bt_dev, const float* guard, bool side = false);

FB_API int32_t fb_adam_step(fb_ctx* ctx, void* stream_, int32_t ntensors, float* const* w_host,
                            const float* const* g_host, float* const* m_host, float* const* v_host,
                            const int64_t* counts_host, float eta, float beta1, float beta2, float eps, float b1t,
                            float b2t, float grad_scale) {
  FB_CHECK_CTX(ctx);
  return adam_common(ctx, (cudaStream_t)stream_, ntensors, w_host, g_host, m_host, v_host, counts_host, eta, beta1, beta2, eps,
                     b1t, b2t, grad_scale, nullptr, nullptr);
}

FB_API int32_t fb_adam_step_dev(fb_ctx* ctx, void* stream_, int32_t ntensors, float* const* w_host,
                                const float* const* g_host, float* const* m_host, float* const* v_host,
                                const int64_t* counts_host, float eta, float beta1, float beta2, float eps,
                                const float* bt_dev, const float* guard_dev, float grad_scale) {
  FB_CHECK_CTX(ctx);
  FB_REQUIRE(bt_dev != nullptr, FB_ERR_INVALID_ARG, "fb_adam_step_dev: bt_dev is NULL");
  return adam_common(ctx, (cudaStream_t)stream_, ntensors, w_host, g_host, m_host, v_host, counts_host, eta, beta1, beta2, eps,
                     0.0f, 0.0f, grad_scale, bt_dev, guard_dev);
}

FB_API int32_t fb_adam_block_dev(fb_ctx* ctx, void* stream_, float* w, const float* g, float* m, float* v, int64_t count, float eta,
                                 float beta1, float beta2, float eps, const float* bt_dev, const float* guard_dev, float grad_scale) {
  FB_CHECK_CTX(ctx);
  FB_REQUIRE(bt_dev != nullptr, FB_ERR_INVALID_ARG, "fb_adam_block_dev: bt_dev is NULL");
  return adam_common(ctx, (cudaStream_t)stream_, 1, &w, &g, &m, &v, &count, eta, beta1, beta2, eps, 0.0f, 0.0f, grad_scale, bt_dev,
                     guard_dev, true);
}

__global__ void adam_advance_kernel(float* __restrict__ bt, float beta1, float beta2, const float* __restrict__ guard) {
  if (guard != nullptr && !isfinite(*guard)) return;
  bt[0] *= beta1;
  bt[1] *= beta2;
}

FB_API int32_t fb_adam_advance(fb_ctx* ctx, void* stream_, float* bt_dev, float beta1, float beta2, const float* guard_dev) {
  FB_CHECK_CTX(ctx);
  FB_REQUIRE(bt_dev != nullptr, FB_ERR_INVALID_ARG, "fb_adam_advance: bt_dev is NULL");
  adam_advance_kernel<<<1, 1, 0, (cudaStream_t)stream_>>>(bt_dev, beta1, beta2, guard_dev);
  FB_LAUNCH_CHECK();
  return FB_OK;
}

static int32_t adam_common(fb_ctx* ctx, cudaStream_t stream, int32_t ntensors, float* const* w_host,
                           const float* const* g_host, float* const* m_host, float* const* v_host,
                           const int64_t* counts_host, float eta, float beta1, float beta2, float eps, float b1t,
                           float b2t, float grad_scale, const float* bt_dev, const float* guard, bool side) {
  FB_REQUIRE(ntensors >= 0, FB_ERR_INVALID_ARG, "fb_adam_step: negative tensor count");
  if (ntensors == 0) return FB_OK;
  FB_REQUIRE(w_host && g_host && m_host && v_host && counts_host, FB_ERR_INVALID_ARG, "fb_adam_step: NULL table");
  // bias corrections in the parameter eltype (Float32), as the rule computes them
  const float inv_c1 = 1.0f / (1.0f - b1t), inv_c2 = 1.0f / (1.0f - b2t);
  int done = 0;
  while (done < ntensors) {
    AdamTable tab;
    memset(&tab, 0, sizeof(tab));
    int k = 0, blocks = 0;
    while (done < ntensors && k < ADAM_MAX_TENSORS) {
      const int64_t cnt = counts_host[done];
      FB_REQUIRE(cnt >= 0, FB_ERR_INVALID_ARG, "fb_adam_step: negative element count for leaf %d", done);
      if (cnt > 0) {
        FB_REQUIRE(w_host[done] && g_host[done] && m_host[done] && v_host[done], FB_ERR_INVALID_ARG,
                   "fb_adam_step: NULL pointer for leaf %d", done);
        const int64_t nb = (cnt + ADAM_CHUNK - 1) / ADAM_CHUNK;
        if ((int64_t)blocks + nb > 0x3fffffff) break;
        tab.w[k] = w_host[done]; tab.g[k] = g_host[done]; tab.m[k] = m_host[done]; tab.v[k] = v_host[done];
        tab.count[k] = cnt;
        tab.block_start[k] = blocks;
        blocks += (int)nb;
        ++k;
      }
      ++done;
    }
    if (k == 0) continue;
    tab.block_start[k] = blocks;
    tab.ntensors = k;
    if (side)
      adam_kernel<ADAM_SIDE_THREADS, 2048 / ADAM_SIDE_THREADS><<<(unsigned)blocks, ADAM_SIDE_THREADS, 0, stream>>>(
          tab, eta, beta1, beta2, eps, inv_c1, inv_c2, grad_scale, bt_dev, guard);
    else
      adam_kernel<EW_THREADS, 1><<<(unsigned)blocks, EW_THREADS, 0, stream>>>(tab, eta, beta1, beta2, eps, inv_c1, inv_c2, grad_scale,
                                                                              bt_dev, guard);
    FB_LAUNCH_CHECK();
  }
  return FB_OK;
}
