// Gradient exchange over peer memory: the copy-engine form of reduce-scatter and all-gather for the data-parallel
// step with a sharded optimiser.
//
// Every rank owns 1/N of each gradient bucket.  Instead of NCCL's reduce-scatter and all-gather kernels - which hold
// SMs while the reverse sweep's GEMMs want all of them - the blocks travel as plain device-to-device copies into
// buffers the peers have mapped (CUDA IPC, NVLink / NVSwitch; the copies run on the copy engines):
//   1. my block p of the bucket -> slot [me] of peer p's staging area, for every peer p   (fb_peer_scatter_blocks)
//   2. a one-element NCCL all-reduce on the same stream as a barrier: when it completes here, every peer's copies
//      (ordered before its barrier kernel in its stream) have landed in my staging area
//   3. mean over the N slots in rank order, then Adam on my block                           (fb_reduce_slots)
//   4. my updated parameter block -> its place in every peer's parameter buffer            (fb_peer_gather_block)
// and one more barrier at the end of the step, before anybody reads the parameters again.  The sums run in a fixed
// order, so every run and every rank count gives bitwise reproducible averages.
#include "common.cuh"

namespace {

constexpr int PEER_MAX_RANKS = 16;
struct SlotTable { const float* p[PEER_MAX_RANKS]; };

__global__ void __launch_bounds__(256)
reduce_slots_kernel(SlotTable t, int nslots, float* __restrict__ out, int64_t count4, int64_t count, float scale) {
  const int64_t stride = (int64_t)gridDim.x * 256;
  for (int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x; i < count4; i += stride) {
    float4 a = __ldcs((const float4*)t.p[0] + i);
    for (int s = 1; s < nslots; ++s) {
      const float4 b = __ldcs((const float4*)t.p[s] + i);
      a.x += b.x; a.y += b.y; a.z += b.z; a.w += b.w;
    }
    a.x *= scale; a.y *= scale; a.z *= scale; a.w *= scale;
    ((float4*)out)[i] = a;
  }
  // tail (count not a multiple of 4)
  for (int64_t i = 4 * count4 + (int64_t)blockIdx.x * 256 + threadIdx.x; i < count; i += stride) {
    float a = t.p[0][i];
    for (int s = 1; s < nslots; ++s) a += t.p[s][i];
    out[i] = a * scale;
  }
}

// Copies to different peers are issued on different auxiliary streams so that several copy engines work at once
// (one stream's copies run one after the other and reach less than half of the NVLink bandwidth).  The fork / join
// events make the auxiliary work part of the caller's stream order, also under stream capture.  The pool is created
// by fb_peer_alloc, outside any capture.
constexpr int PEER_AUX = 8;
constexpr int PEER_MAX_DEVICES = 64;
struct PeerPool {
  bool ready = false;
  cudaStream_t aux[PEER_AUX];
  cudaEvent_t fork, join[PEER_AUX];
};
PeerPool g_peer_pool[PEER_MAX_DEVICES];

int32_t peer_pool_create(int device) {
  if (device < 0 || device >= PEER_MAX_DEVICES) return fb_fail(FB_ERR_UNSUPPORTED, "peer exchange: device index %d not supported", device);
  PeerPool& pp = g_peer_pool[device];
  if (pp.ready) return FB_OK;
  int lo = 0, hi = 0;
  FB_CUDA(cudaDeviceGetStreamPriorityRange(&lo, &hi));
  for (int i = 0; i < PEER_AUX; ++i) {
    FB_CUDA(cudaStreamCreateWithPriority(&pp.aux[i], cudaStreamNonBlocking, hi));
    FB_CUDA(cudaEventCreateWithFlags(&pp.join[i], cudaEventDisableTiming));
  }
  FB_CUDA(cudaEventCreateWithFlags(&pp.fork, cudaEventDisableTiming));
  pp.ready = true;
  return FB_OK;
}

// copies[i] = (dst, src) for i < n, all of `bytes` bytes: spread over the auxiliary streams, joined back into `stream`
int32_t peer_parallel_copies(fb_ctx* ctx, cudaStream_t stream, int n, float* const* dst, const float* const* src, size_t bytes) {
  PeerPool& pp = g_peer_pool[ctx->device];
  if (!pp.ready) {
    for (int i = 0; i < n; ++i) FB_CUDA(cudaMemcpyAsync(dst[i], src[i], bytes, cudaMemcpyDeviceToDevice, stream));
    return FB_OK;
  }
  FB_CUDA(cudaEventRecord(pp.fork, stream));
  const int used = n < PEER_AUX ? n : PEER_AUX;
  for (int a = 0; a < used; ++a) FB_CUDA(cudaStreamWaitEvent(pp.aux[a], pp.fork, 0));
  for (int i = 0; i < n; ++i) FB_CUDA(cudaMemcpyAsync(dst[i], src[i], bytes, cudaMemcpyDeviceToDevice, pp.aux[i % PEER_AUX]));
  for (int a = 0; a < used; ++a) {
    FB_CUDA(cudaEventRecord(pp.join[a], pp.aux[a]));
    FB_CUDA(cudaStreamWaitEvent(stream, pp.join[a], 0));
  }
  return FB_OK;
}

}  // namespace

FB_API int32_t fb_peer_alloc(fb_ctx* ctx, int64_t bytes, void** ptr_out, void* handle_host) {
  FB_CHECK_CTX(ctx);
  FB_REQUIRE(ptr_out && handle_host && bytes >= 1, FB_ERR_INVALID_ARG, "fb_peer_alloc: bad arguments");
  *ptr_out = nullptr;
  FB_CUDA(cudaSetDevice(ctx->device));
  const int32_t pst = peer_pool_create(ctx->device);
  if (pst != FB_OK) return pst;
  void* p = nullptr;
  cudaError_t e = cudaMalloc(&p, (size_t)bytes);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return fb_fail(FB_ERR_ALLOC, "fb_peer_alloc: cudaMalloc(%lld) failed: %s", (long long)bytes, cudaGetErrorString(e));
  }
  cudaIpcMemHandle_t h;
  e = cudaIpcGetMemHandle(&h, p);
  if (e != cudaSuccess) {
    cudaGetLastError();
    cudaFree(p);
    return fb_fail(FB_ERR_CUDA, "fb_peer_alloc: cudaIpcGetMemHandle failed: %s", cudaGetErrorString(e));
  }
  static_assert(sizeof(cudaIpcMemHandle_t) == FB_PEER_HANDLE_BYTES, "IPC handle size");
  memcpy(handle_host, &h, sizeof(h));
  FB_CUDA(cudaMemset(p, 0, (size_t)bytes));
  *ptr_out = p;
  return FB_OK;
}

FB_API int32_t fb_peer_open(fb_ctx* ctx, const void* handle_host, void** ptr_out) {
  FB_CHECK_CTX(ctx);
  FB_REQUIRE(ptr_out && handle_host, FB_ERR_INVALID_ARG, "fb_peer_open: NULL pointer");
  *ptr_out = nullptr;
  FB_CUDA(cudaSetDevice(ctx->device));
  cudaIpcMemHandle_t h;
  memcpy(&h, handle_host, sizeof(h));
  void* p = nullptr;
  const cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return fb_fail(FB_ERR_CUDA, "fb_peer_open: cudaIpcOpenMemHandle failed: %s", cudaGetErrorString(e));
  }
  *ptr_out = p;
  return FB_OK;
}

FB_API int32_t fb_peer_close(fb_ctx* ctx, void* ptr) {
  FB_CHECK_CTX(ctx);
  if (ptr == nullptr) return FB_OK;
  FB_CUDA(cudaIpcCloseMemHandle(ptr));
  return FB_OK;
}

FB_API int32_t fb_peer_free(fb_ctx* ctx, void* ptr) {
  FB_CHECK_CTX(ctx);
  if (ptr == nullptr) return FB_OK;
  FB_CUDA(cudaFree(ptr));
  return FB_OK;
}

FB_API int32_t fb_peer_scatter_blocks(fb_ctx* ctx, void* stream, const float* bucket, float* const* peer_stage_host, int32_t nranks,
                                      int32_t rank, int64_t blk) {
  FB_CHECK_CTX(ctx);
  FB_REQUIRE(bucket && peer_stage_host && nranks >= 2 && nranks <= PEER_MAX_RANKS && rank >= 0 && rank < nranks && blk >= 1,
             FB_ERR_INVALID_ARG, "fb_peer_scatter_blocks: bad arguments (ranks %d, rank %d, block %lld)", nranks, rank, (long long)blk);
  float* dst[PEER_MAX_RANKS];
  const float* src[PEER_MAX_RANKS];
  for (int i = 1; i < nranks; ++i) {
    const int p = (rank + i) % nranks;     // every rank starts with a different peer
    FB_REQUIRE(peer_stage_host[p] != nullptr, FB_ERR_INVALID_ARG, "fb_peer_scatter_blocks: peer %d has no staging pointer", p);
    dst[i - 1] = peer_stage_host[p] + (int64_t)rank * blk;
    src[i - 1] = bucket + (int64_t)p * blk;
  }
  return peer_parallel_copies(ctx, (cudaStream_t)stream, nranks - 1, dst, src, (size_t)blk * sizeof(float));
}

FB_API int32_t fb_peer_gather_block(fb_ctx* ctx, void* stream, const float* my_block, float* const* peer_dst_host, int32_t nranks,
                                    int32_t rank, int64_t blk) {
  FB_CHECK_CTX(ctx);
  FB_REQUIRE(my_block && peer_dst_host && nranks >= 2 && nranks <= PEER_MAX_RANKS && rank >= 0 && rank < nranks && blk >= 1,
             FB_ERR_INVALID_ARG, "fb_peer_gather_block: bad arguments (ranks %d, rank %d, block %lld)", nranks, rank, (long long)blk);
  float* dst[PEER_MAX_RANKS];
  const float* src[PEER_MAX_RANKS];
  for (int i = 1; i < nranks; ++i) {
    const int p = (rank + i) % nranks;
    FB_REQUIRE(peer_dst_host[p] != nullptr, FB_ERR_INVALID_ARG, "fb_peer_gather_block: peer %d has no destination pointer", p);
    dst[i - 1] = peer_dst_host[p];
    src[i - 1] = my_block;
  }
  return peer_parallel_copies(ctx, (cudaStream_t)stream, nranks - 1, dst, src, (size_t)blk * sizeof(float));
}

FB_API int32_t fb_reduce_slots(fb_ctx* ctx, void* stream, int32_t nslots, const float* const* slots_host, float* out, int64_t count,
                               float scale) {
  FB_CHECK_CTX(ctx);
  FB_REQUIRE(slots_host && out && nslots >= 1 && nslots <= PEER_MAX_RANKS && count >= 0, FB_ERR_INVALID_ARG, "fb_reduce_slots: bad arguments");
  if (count == 0) return FB_OK;
  SlotTable t;
  bool vec = fb_aligned16(out);
  for (int s = 0; s < PEER_MAX_RANKS; ++s) {
    t.p[s] = s < nslots ? slots_host[s] : nullptr;
    if (s < nslots) {
      FB_REQUIRE(slots_host[s] != nullptr, FB_ERR_INVALID_ARG, "fb_reduce_slots: slot %d is NULL", s);
      vec = vec && fb_aligned16(slots_host[s]);
    }
  }
  const int64_t count4 = vec ? count / 4 : 0;
  int64_t blocks = (count / 4 + 255) / 256 + 1;
  if (blocks > (int64_t)ctx->sm_count * 8) blocks = (int64_t)ctx->sm_count * 8;
  reduce_slots_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(t, nslots, out, count4, count, scale);
  FB_LAUNCH_CHECK();
  return FB_OK;
}
