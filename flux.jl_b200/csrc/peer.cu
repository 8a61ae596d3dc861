// Gradient exchange over peer memory for the data-parallel step with a sharded optimiser (single node, NVLink /
// NVSwitch): reduce-scatter and all-gather as small kernels that STORE into buffers the peers have mapped.
//
// Every rank owns 1/N of each gradient bucket.  A staging area, the parameter buffer and a page of barrier words of
// every rank are allocated by fb_peer_alloc and mapped by all the others (CUDA IPC).  Per bucket:
//   1. fb_peer_push_blocks: block p of my gradients -> slot [me] of peer p's staging area, for every peer p
//   2. fb_peer_barrier: one warp writes this rank's epoch into a flag word of every peer and waits (bounded) until
//      every peer's epoch has arrived here: the peers' blocks have landed in my staging area
//   3. fb_reduce_slots: mean over the N slots of my block in rank order (local reads), then Adam on my block
//   4. fb_peer_push_blocks: my updated block -> its place in every peer's parameter buffer, behind a barrier that
//      says every rank has stopped reading the old values; one more barrier before anybody reads the new ones.
//      With deferred gathers step 4 runs at the start of the next step, beside its forward pass.
// Stores over NVLink are posted, so a few warps per SM keep the links busy; loads from a peer would need far more
// bytes in flight than the registers beside a resident GEMM CTA allow (measured: 150 GB/s pulling, 8 ranks).
// All kernels here are "side kernels": 128 threads of at most 32 registers, see SIDE_THREADS.  NCCL's kernels do
// not fit beside the GEMM and wait for it to end; they remain the path when the ranks cannot map each other's memory.
// The sums run in rank order, so every run gives bitwise the same averages.
#include "common.cuh"

namespace {

constexpr int PEER_MAX_RANKS = 16;
struct SlotTable { const float* p[PEER_MAX_RANKS]; };

// Side-kernel shape: 128 threads of at most 32 registers.  A resident 3xTF32 GEMM CTA (22 warps of 80 registers) leaves
// about 1 K registers free in each of the SM's four register-file partitions: one warp of 32 registers per partition
// still fits, a wider CTA or a fatter thread waits until the GEMM has ended.
constexpr int SIDE_THREADS = 128;

__global__ void __launch_bounds__(SIDE_THREADS, 2048 / SIDE_THREADS)
reduce_slots_kernel(const __grid_constant__ SlotTable t, int nslots, float* __restrict__ out, int64_t count4, int64_t count, float scale) {
  const int64_t stride = (int64_t)gridDim.x * SIDE_THREADS;
  for (int64_t i = (int64_t)blockIdx.x * SIDE_THREADS + threadIdx.x; i < count4; i += stride) {
    float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int s0 = 0; s0 < nslots; s0 += 4) {
      float4 v[4];
#pragma unroll
      for (int s = 0; s < 4; ++s)        // the loads of a group are issued before the first sum waits for one
        if (s0 + s < nslots) v[s] = __ldcs((const float4*)t.p[s0 + s] + i);
#pragma unroll
      for (int s = 0; s < 4; ++s)
        if (s0 + s < nslots) { a.x += v[s].x; a.y += v[s].y; a.z += v[s].z; a.w += v[s].w; }
    }
    a.x *= scale; a.y *= scale; a.z *= scale; a.w *= scale;
    ((float4*)out)[i] = a;
  }
  // tail (count not a multiple of 4, or a pointer off the 16-byte grid)
  for (int64_t i = 4 * count4 + (int64_t)blockIdx.x * SIDE_THREADS + threadIdx.x; i < count; i += stride) {
    float a = 0.f;
    for (int s = 0; s < nslots; ++s) a += t.p[s][i];
    out[i] = a * scale;
  }
}

// Barrier between the ranks of one node.  flags.p[r] = rank r's array of nranks epoch words (this rank's own array is
// local memory, the others are mapped).  `epoch` is a device word owned by this rank that counts the barriers passed,
// so that a captured launch works for every replay.  Lane r posts to peer r and waits for peer r.  A wait that runs
// out (a peer that died or never reached the barrier) writes FB_DEV_ERR_PEER_BARRIER to the device error word and
// lets the kernel end: the context stays usable and the host finds the code with fb_device_error.
constexpr int32_t FB_DEV_ERR_PEER_BARRIER = 9101;

struct FlagTable { uint32_t* p[PEER_MAX_RANKS]; };

__global__ void __maxnreg__(32)
peer_barrier_kernel(const __grid_constant__ FlagTable flags, int nranks, int rank, uint32_t* __restrict__ epoch, int32_t* __restrict__ dev_err, uint64_t limit_ns) {
  const int lane = threadIdx.x;
  const uint32_t e = *epoch + 1u;
  __syncwarp();
  if (lane < nranks && lane != rank) {
    uint32_t* remote = flags.p[lane] + rank;
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(remote), "r"(e) : "memory");
    const uint32_t* mine = flags.p[rank] + lane;
    uint64_t t0;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
    uint32_t polls = 0;
    while (true) {
      uint32_t seen;
      asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(mine) : "memory");
      if ((int32_t)(seen - e) >= 0) break;
      if ((++polls & 63u) == 0) {
        uint64_t t1;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t1));
        if (t1 - t0 > limit_ns) { atomicCAS(dev_err, 0, FB_DEV_ERR_PEER_BARRIER); break; }
      }
      __nanosleep(64);
    }
  }
  __syncwarp();
  if (lane == 0) *epoch = e;
}

// blockIdx.y selects the peer (starting behind this rank, so that the ranks do not all write to the same one first);
// every thread moves four 16-byte words per round, loaded (locally) together before the first (remote) store.
__global__ void __launch_bounds__(SIDE_THREADS, 2048 / SIDE_THREADS)
push_blocks_kernel(const __grid_constant__ SlotTable dst, const float* __restrict__ src, int64_t src_stride, int nranks, int rank,
                   int64_t blk4, int64_t blk) {
  const int r = (rank + 1 + (int)blockIdx.y) % nranks;
  const float* s = src + (int64_t)r * src_stride;
  float* d = const_cast<float*>(dst.p[r]);
  const int64_t round = (int64_t)gridDim.x * (4 * SIDE_THREADS);
  for (int64_t base = (int64_t)blockIdx.x * (4 * SIDE_THREADS) + threadIdx.x; base < blk4; base += round) {
    float4 v[4];
#pragma unroll
    for (int k = 0; k < 4; ++k)
      if (base + k * SIDE_THREADS < blk4) v[k] = __ldcs((const float4*)s + base + k * SIDE_THREADS);
#pragma unroll
    for (int k = 0; k < 4; ++k)
      if (base + k * SIDE_THREADS < blk4) ((float4*)d)[base + k * SIDE_THREADS] = v[k];
  }
  for (int64_t i = 4 * blk4 + (int64_t)blockIdx.x * SIDE_THREADS + threadIdx.x; i < blk; i += (int64_t)gridDim.x * SIDE_THREADS) d[i] = s[i];
}

}  // namespace

int32_t fb_side_kernels_prepare_peer() {
  FB_CUDA(cudaFuncSetAttribute(reduce_slots_kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared));
  FB_CUDA(cudaFuncSetAttribute(push_blocks_kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared));
  FB_CUDA(cudaFuncSetAttribute(peer_barrier_kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared));
  return FB_OK;
}

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

FB_API int32_t fb_peer_barrier(fb_ctx* ctx, void* stream, uint32_t* const* peer_flags_host, int32_t nranks, int32_t rank,
                               uint32_t* epoch_dev, int64_t timeout_ms) {
  FB_CHECK_CTX(ctx);
  FB_REQUIRE(peer_flags_host && epoch_dev && nranks >= 2 && nranks <= PEER_MAX_RANKS && rank >= 0 && rank < nranks && timeout_ms >= 1,
             FB_ERR_INVALID_ARG, "fb_peer_barrier: bad arguments (ranks %d, rank %d, timeout %lld ms)", nranks, rank, (long long)timeout_ms);
  FlagTable t;
  for (int p = 0; p < PEER_MAX_RANKS; ++p) {
    t.p[p] = p < nranks ? peer_flags_host[p] : nullptr;
    FB_REQUIRE(p >= nranks || t.p[p] != nullptr, FB_ERR_INVALID_ARG, "fb_peer_barrier: rank %d has no flag array", p);
  }
  peer_barrier_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(t, nranks, rank, epoch_dev, ctx->dev_error, (uint64_t)timeout_ms * 1000000ull);
  FB_LAUNCH_CHECK();
  return FB_OK;
}

FB_API int32_t fb_peer_push_blocks(fb_ctx* ctx, void* stream, const float* src, int64_t src_stride, float* const* peer_dst_host,
                                   int32_t nranks, int32_t rank, int64_t blk) {
  FB_CHECK_CTX(ctx);
  FB_REQUIRE(src && peer_dst_host && nranks >= 2 && nranks <= PEER_MAX_RANKS && rank >= 0 && rank < nranks && blk >= 1 && src_stride >= 0,
             FB_ERR_INVALID_ARG, "fb_peer_push_blocks: bad arguments (ranks %d, rank %d, block %lld)", nranks, rank, (long long)blk);
  SlotTable t;
  bool vec = fb_aligned16(src) && blk % 4 == 0 && src_stride % 4 == 0;
  for (int p = 0; p < PEER_MAX_RANKS; ++p) {
    t.p[p] = (p < nranks && p != rank) ? peer_dst_host[p] : nullptr;
    if (p < nranks && p != rank) {
      FB_REQUIRE(peer_dst_host[p] != nullptr, FB_ERR_INVALID_ARG, "fb_peer_push_blocks: peer %d has no destination pointer", p);
      vec = vec && fb_aligned16(peer_dst_host[p]);
    }
  }
  const int64_t blk4 = vec ? blk / 4 : 0;
  int64_t per_peer = (blk / 4 + 4 * SIDE_THREADS - 1) / (4 * SIDE_THREADS) + 1;
  // (grids twice as large were measured slower at 2 and at 8 GPUs: 19.6 vs 18.2-18.6 ms and 6.12 vs 5.91 ms per step)
  const int64_t cap = ((int64_t)ctx->sm_count * 2 + nranks - 2) / (nranks - 1);
  if (per_peer > cap) per_peer = cap;
  push_blocks_kernel<<<dim3((unsigned)per_peer, (unsigned)(nranks - 1)), SIDE_THREADS, 0, (cudaStream_t)stream>>>(t, src, src_stride, nranks,
                                                                                                                 rank, blk4, blk);
  FB_LAUNCH_CHECK();
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
  int64_t blocks = (count / 4 + SIDE_THREADS - 1) / SIDE_THREADS + 1;
  if (blocks > (int64_t)ctx->sm_count * 2) blocks = (int64_t)ctx->sm_count * 2;
  reduce_slots_kernel<<<(unsigned)blocks, SIDE_THREADS, 0, (cudaStream_t)stream>>>(t, nslots, out, count4, count, scale);
  FB_LAUNCH_CHECK();
  return FB_OK;
}
