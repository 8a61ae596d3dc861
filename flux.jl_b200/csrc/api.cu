// Context, error reporting and device-memory entry points of libfluxb200.
#include <stdarg.h>

#include "common.cuh"

static thread_local char g_last_error[512] = "";

void fb_set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_last_error, sizeof(g_last_error), fmt, ap);
  va_end(ap);
}

int32_t fb_fail(int32_t code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_last_error, sizeof(g_last_error), fmt, ap);
  va_end(ap);
  return code;
}

unsigned long long g_fb_kernel_launches = 0;

FB_API int32_t fb_version(void) { return FB_VERSION; }

FB_API int64_t fb_kernel_launches(void) { return (int64_t)g_fb_kernel_launches; }

FB_API const char* fb_last_error(void) { return g_last_error; }

FB_API int32_t fb_ctx_create(int32_t device, fb_ctx** out) {
  FB_REQUIRE(out != nullptr, FB_ERR_INVALID_ARG, "fb_ctx_create: out is NULL");
  *out = nullptr;
  int count = 0;
  cudaError_t e = cudaGetDeviceCount(&count);
  if (e != cudaSuccess || count == 0)
    return fb_fail(FB_ERR_CUDA, "fb_ctx_create: no CUDA device available (%s); this library has no CPU fallback",
                   cudaGetErrorString(e));
  FB_REQUIRE(device >= 0 && device < count, FB_ERR_INVALID_ARG, "fb_ctx_create: device %d out of range [0,%d)",
             device, count);
  FB_CUDA(cudaSetDevice(device));
  cudaDeviceProp prop;
  FB_CUDA(cudaGetDeviceProperties(&prop, device));
  if (prop.major != 10)
    return fb_fail(FB_ERR_UNSUPPORTED, "fb_ctx_create: device %d is sm_%d%d; this library is built for sm_100a only",
                   device, prop.major, prop.minor);
  fb_ctx* c = new fb_ctx();
  c->device = device;
  c->sm_count = prop.multiProcessorCount;
  c->reserved_sms = 0;
  c->smem_optin = prop.sharedMemPerBlockOptin;
  c->scratch = nullptr;
  c->scratch_bytes = 0;
  c->retired_count = 0;
  c->dev_error = nullptr;
  c->gemm_ws = nullptr;
  e = cudaMalloc(&c->dev_error, 256);
  if (e != cudaSuccess) {
    delete c;
    return fb_fail(FB_ERR_ALLOC, "fb_ctx_create: cudaMalloc failed: %s", cudaGetErrorString(e));
  }
  cudaMemset(c->dev_error, 0, 256);
  int32_t ws_status = fb_side_kernels_prepare_elementwise();
  if (ws_status == FB_OK) ws_status = fb_side_kernels_prepare_peer();
  if (ws_status == FB_OK) ws_status = fb_gemm_workspace_create(c);
  if (ws_status != FB_OK) {
    cudaFree(c->dev_error);
    delete c;
    return ws_status;
  }
  *out = c;
  return FB_OK;
}

FB_API int32_t fb_ctx_set_reserved_sms(fb_ctx* ctx, int32_t n) {
  FB_CHECK_CTX(ctx);
  FB_REQUIRE(n >= 0 && n <= ctx->sm_count - 2, FB_ERR_INVALID_ARG, "fb_ctx_set_reserved_sms: %d is outside [0, %d]", n,
             ctx->sm_count - 2);
  ctx->reserved_sms = n;
  return FB_OK;
}

FB_API int32_t fb_ctx_destroy(fb_ctx* ctx) {
  if (ctx == nullptr) return FB_OK;
  cudaSetDevice(ctx->device);
  cudaDeviceSynchronize();
  if (ctx->scratch) cudaFree(ctx->scratch);
  for (int i = 0; i < ctx->retired_count; ++i) cudaFree(ctx->retired[i]);
  if (ctx->dev_error) cudaFree(ctx->dev_error);
  fb_gemm_workspace_destroy(ctx);
  delete ctx;
  return FB_OK;
}

void* fb_scratch(fb_ctx* ctx, cudaStream_t stream, size_t bytes) {
  (void)stream;
  if (bytes <= ctx->scratch_bytes && ctx->scratch != nullptr) return ctx->scratch;
  // grow geometrically; the outgrown block stays allocated until the context is destroyed, because work already
  // enqueued - or captured in a CUDA graph - may still name it
  size_t want = bytes < (size_t(1) << 22) ? (size_t(1) << 22) : bytes;
  if (want < 2 * ctx->scratch_bytes) want = 2 * ctx->scratch_bytes;
  want = (want + 255) & ~size_t(255);
  void* p = nullptr;
  if (cudaMalloc(&p, want) != cudaSuccess) {
    cudaGetLastError();
    fb_set_error("scratch arena: cudaMalloc of %zu bytes failed", want);
    return nullptr;
  }
  if (ctx->scratch != nullptr && ctx->retired_count < FB_MAX_RETIRED) ctx->retired[ctx->retired_count++] = ctx->scratch;
  ctx->scratch = p;
  ctx->scratch_bytes = want;
  return p;
}

FB_API int32_t fb_malloc(fb_ctx* ctx, int64_t bytes, void** out) {
  FB_CHECK_CTX(ctx);
  FB_REQUIRE(out != nullptr && bytes >= 0, FB_ERR_INVALID_ARG, "fb_malloc: bad arguments");
  *out = nullptr;
  if (bytes == 0) return FB_OK;
  cudaError_t e = cudaMalloc(out, (size_t)bytes);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return fb_fail(FB_ERR_ALLOC, "fb_malloc: cudaMalloc(%lld) failed: %s", (long long)bytes, cudaGetErrorString(e));
  }
  return FB_OK;
}

FB_API int32_t fb_free(fb_ctx* ctx, void* ptr) {
  FB_CHECK_CTX(ctx);
  if (ptr == nullptr) return FB_OK;
  FB_CUDA(cudaFree(ptr));
  return FB_OK;
}

FB_API int32_t fb_memcpy_h2d(fb_ctx* ctx, void* stream, void* dst, const void* src_host, int64_t bytes) {
  FB_CHECK_CTX(ctx);
  FB_REQUIRE(bytes >= 0, FB_ERR_INVALID_ARG, "fb_memcpy_h2d: negative size");
  if (bytes == 0) return FB_OK;
  FB_REQUIRE(dst && src_host, FB_ERR_INVALID_ARG, "fb_memcpy_h2d: NULL pointer");
  FB_CUDA(cudaMemcpyAsync(dst, src_host, (size_t)bytes, cudaMemcpyHostToDevice, (cudaStream_t)stream));
  return FB_OK;
}

FB_API int32_t fb_memcpy_d2h(fb_ctx* ctx, void* stream, void* dst_host, const void* src, int64_t bytes) {
  FB_CHECK_CTX(ctx);
  FB_REQUIRE(bytes >= 0, FB_ERR_INVALID_ARG, "fb_memcpy_d2h: negative size");
  if (bytes == 0) return FB_OK;
  FB_REQUIRE(dst_host && src, FB_ERR_INVALID_ARG, "fb_memcpy_d2h: NULL pointer");
  FB_CUDA(cudaMemcpyAsync(dst_host, src, (size_t)bytes, cudaMemcpyDeviceToHost, (cudaStream_t)stream));
  FB_CUDA(cudaStreamSynchronize((cudaStream_t)stream));
  return FB_OK;
}

FB_API int32_t fb_memcpy_d2d(fb_ctx* ctx, void* stream, void* dst, const void* src, int64_t bytes) {
  FB_CHECK_CTX(ctx);
  FB_REQUIRE(bytes >= 0, FB_ERR_INVALID_ARG, "fb_memcpy_d2d: negative size");
  if (bytes == 0) return FB_OK;
  FB_REQUIRE(dst && src, FB_ERR_INVALID_ARG, "fb_memcpy_d2d: NULL pointer");
  FB_CUDA(cudaMemcpyAsync(dst, src, (size_t)bytes, cudaMemcpyDeviceToDevice, (cudaStream_t)stream));
  return FB_OK;
}

FB_API int32_t fb_memset(fb_ctx* ctx, void* stream, void* dst, int32_t byte_value, int64_t bytes) {
  FB_CHECK_CTX(ctx);
  FB_REQUIRE(bytes >= 0, FB_ERR_INVALID_ARG, "fb_memset: negative size");
  if (bytes == 0) return FB_OK;
  FB_REQUIRE(dst, FB_ERR_INVALID_ARG, "fb_memset: NULL pointer");
  FB_CUDA(cudaMemsetAsync(dst, byte_value, (size_t)bytes, (cudaStream_t)stream));
  return FB_OK;
}

FB_API int32_t fb_sync(fb_ctx* ctx, void* stream) {
  FB_CHECK_CTX(ctx);
  FB_CUDA(cudaStreamSynchronize((cudaStream_t)stream));
  return FB_OK;
}

FB_API int32_t fb_device_error(fb_ctx* ctx, void* stream, int32_t* out_host) {
  FB_CHECK_CTX(ctx);
  FB_REQUIRE(out_host, FB_ERR_INVALID_ARG, "fb_device_error: out is NULL");
  FB_CUDA(cudaMemcpyAsync(out_host, ctx->dev_error, sizeof(int32_t), cudaMemcpyDeviceToHost, (cudaStream_t)stream));
  FB_CUDA(cudaStreamSynchronize((cudaStream_t)stream));
  if (*out_host != 0) {
    // a kernel that gave up may have left GEMM tickets drawn: start the next launch from a clean state
    fb_gemm_workspace_reset(ctx, (cudaStream_t)stream);
    FB_CUDA(cudaMemsetAsync(ctx->dev_error, 0, sizeof(int32_t), (cudaStream_t)stream));
  }
  return FB_OK;
}

// ------------------------------------------------------------------ bounded-wait self test ---
// A one-block kernel that waits, with an iteration limit, on an mbarrier nobody ever arrives on: the wait runs
// out, the kernel records code 9001 in the context's device error word and returns.  It exists so that the host
// side of the failure path (the error word is read, reported and cleared; launches that follow work again) can be
// exercised without any kernel misbehaving.
__global__ void fb_selftest_wait_kernel(int32_t* dev_err, uint32_t polls) {
  __shared__ __align__(8) uint64_t bar;
  const uint32_t b = (uint32_t)__cvta_generic_to_shared(&bar);
  if (threadIdx.x == 0) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(b) : "memory");
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    uint32_t ok = 0;
    for (uint32_t it = 0; it < polls && !ok; ++it)
      asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                   : "=r"(ok) : "r"(b), "r"(0u) : "memory");
    if (!ok) atomicExch(dev_err, 9001);
  }
}

FB_API int32_t fb_selftest_bounded_wait(fb_ctx* ctx, void* stream, int32_t polls) {
  FB_CHECK_CTX(ctx);
  FB_REQUIRE(polls >= 1 && polls <= 4096, FB_ERR_INVALID_ARG, "fb_selftest_bounded_wait: polls must be in [1, 4096]");
  fb_selftest_wait_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(ctx->dev_error, (uint32_t)polls);
  FB_LAUNCH_CHECK();
  return FB_OK;
}
