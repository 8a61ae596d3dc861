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

}  // namespace

FB_API int32_t fb_peer_alloc(fb_ctx* ctx, int64_t bytes, void** ptr_out, void* handle_host) {
  FB_CHECK_CTX(ctx);
  FB_REQUIRE(ptr_out && handle_host && bytes >= 1, FB_ERR_INVALID_ARG, "fb_peer_alloc: bad arguments");
  *ptr_out = nullptr;
  FB_CUDA(cudaSetDevice(ctx->device));
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
  for (int i = 1; i < nranks; ++i) {
    const int p = (rank + i) % nranks;     // every rank starts with a different peer
    FB_REQUIRE(peer_stage_host[p] != nullptr, FB_ERR_INVALID_ARG, "fb_peer_scatter_blocks: peer %d has no staging pointer", p);
    FB_CUDA(cudaMemcpyAsync(peer_stage_host[p] + (int64_t)rank * blk, bucket + (int64_t)p * blk, (size_t)blk * sizeof(float),
                            cudaMemcpyDeviceToDevice, (cudaStream_t)stream));
  }
  return FB_OK;
}

FB_API int32_t fb_peer_gather_block(fb_ctx* ctx, void* stream, const float* my_block, float* const* peer_dst_host, int32_t nranks,
                                    int32_t rank, int64_t blk) {
  FB_CHECK_CTX(ctx);
  FB_REQUIRE(my_block && peer_dst_host && nranks >= 2 && nranks <= PEER_MAX_RANKS && rank >= 0 && rank < nranks && blk >= 1,
             FB_ERR_INVALID_ARG, "fb_peer_gather_block: bad arguments (ranks %d, rank %d, block %lld)", nranks, rank, (long long)blk);
  for (int i = 1; i < nranks; ++i) {
    const int p = (rank + i) % nranks;
    FB_REQUIRE(peer_dst_host[p] != nullptr, FB_ERR_INVALID_ARG, "fb_peer_gather_block: peer %d has no destination pointer", p);
    FB_CUDA(cudaMemcpyAsync(peer_dst_host[p], my_block, (size_t)blk * sizeof(float), cudaMemcpyDeviceToDevice, (cudaStream_t)stream));
  }
  return FB_OK;
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
