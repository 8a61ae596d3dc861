// Tensor-core GEMM for Float32 data on sm_100a: TMA -> shared memory -> tcgen05.mma (TF32, accumulators
// in tensor memory) -> tcgen05.ld epilogue with fused bias / activation / pre-activation store.
//
// fp32 accuracy comes from the error-compensated "3xTF32" scheme: every operand tile is split in shared
// memory into hi = x with the 13 low mantissa bits cleared (exactly representable in TF32) and
// lo = x - hi; the accumulator receives A_lo*B_hi + A_hi*B_lo + A_hi*B_hi in fp32.  The dropped
// lo*lo term is ~2^-22 relative.
//
// One CTA computes one 128 x BN tile of row-major C[M][N]; K is walked in blocks of 16 floats through a
// 4-stage ring.  Warp roles: warp 0 issues TMA loads, warp 1 owns tensor memory and issues the MMAs,
// warps 2-5 split the landed tiles into hi / lo and afterwards run the epilogue (one TMEM lane quadrant
// each).  Operands may be K-major (k contiguous) or MN-major (m / n contiguous) in global memory; the
// shared-memory layouts are the canonical ones the MMA descriptors name: 64-byte swizzle for K-major tiles
// (8 rows x 64 B atoms) and, for MN-major tiles, the 128-byte swizzle with 32-byte atoms (128 B x 4 k-rows
// per atom), which is the only MN-major layout the tensor core accepts for 32-bit operands.
//
// The tensor core adds into its fp32 accumulator with truncation, so a long K chain drifts (about 3e-5 of
// max|C| at K = 4096).  K is therefore cut into segments of 2048: after each segment the epilogue warps drain
// tensor memory into C with round-to-nearest adds and the next segment starts from a zeroed accumulator.
//
// Every mbarrier wait is bounded; when a wait runs out the kernel records a code in the context's
// device error word, every role leaves its loop, tensor memory is released and the kernel returns.
#include <cuda.h>

#include "common.cuh"

namespace {

constexpr int BM = 128;
constexpr int BK = 16;               // floats per k-block (64 bytes)
constexpr int STAGES = 4;
constexpr int NUM_THREADS = 192;     // 6 warps
constexpr uint32_t WAIT_LIMIT = 1u << 20;
constexpr int SEG_KB = 128;          // k-blocks per accumulation segment (2048 k-values)

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
// Bounded wait.  Returns false when the wait ran out or another role already gave up.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* s_abort) {
  for (uint32_t it = 0; it < WAIT_LIMIT; ++it) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    if (ok) return true;
    if ((it & 255u) == 255u && *s_abort != 0) return false;
  }
  *s_abort = 1;
  return false;
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(bar)
      : "memory");
}

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ void tc_mma_tf32(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                            uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, {%5, %6, %7, %8}, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(0u), "r"(0u), "r"(0u), "r"(0u)
      : "memory");
}

__device__ __forceinline__ void tc_ld_32x32b_x32(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor (sm_100 format: version 1 at bit 46, swizzle mode in bits 61-63).
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes,
                                                   uint32_t layout_type) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr >> 4) & 0x3fffu);
  d |= (uint64_t)((lbo_bytes >> 4) & 0x3fffu) << 16;
  d |= (uint64_t)((sbo_bytes >> 4) & 0x3fffu) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)(layout_type & 7u) << 61;
  return d;
}
constexpr uint32_t LAYOUT_SW128_32B = 1, LAYOUT_SW64 = 4;   // MN-major 32-bit operands only exist in the 32-byte-atom 128B swizzle

template <int BN, int PASSES>
struct Cfg {
  static constexpr int A_BYTES = BM * BK * 4;   // 8 KB
  static constexpr int B_BYTES = BN * BK * 4;   // 16 KB at BN = 256
  static constexpr int STAGE_BYTES = (PASSES == 3 ? 2 : 1) * (A_BYTES + B_BYTES);
  static constexpr int BAR_OFFSET = STAGES * STAGE_BYTES;
  static constexpr int SMEM_BYTES = BAR_OFFSET + 256 + 1024;  // barriers + alignment slack
};

template <bool A_MN, bool B_MN, int BN, int PASSES>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
               float* __restrict__ C, int64_t ldc, float* __restrict__ Z, const float* __restrict__ bias_n, int M,
               int N, int K, int act, int accumulate, int32_t* __restrict__ dev_err) {
  using cfg = Cfg<BN, PASSES>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const uint32_t smem_base = smem_u32(smem);
  uint64_t* bars = (uint64_t*)(smem + cfg::BAR_OFFSET);
  const uint32_t bar_base = smem_base + cfg::BAR_OFFSET;
  // barrier slots: full[0..S), ready[S..2S), empty[2S..3S), tmem_full[3S], tmem_empty[3S+1]
  auto full_bar = [&](int s) { return bar_base + 8u * (uint32_t)s; };
  auto ready_bar = [&](int s) { return bar_base + 8u * (uint32_t)(STAGES + s); };
  auto empty_bar = [&](int s) { return bar_base + 8u * (uint32_t)(2 * STAGES + s); };
  const uint32_t tmem_full_bar = bar_base + 8u * (uint32_t)(3 * STAGES);
  const uint32_t tmem_empty_bar = bar_base + 8u * (uint32_t)(3 * STAGES + 1);
  volatile uint32_t* s_tmem = (volatile uint32_t*)(bars + 3 * STAGES + 2);
  volatile int* s_abort = (volatile int*)(bars + 3 * STAGES + 3);

  // a wait that ran out earlier (in this or a previous launch) leaves the error word set: do not start
  __shared__ int s_skip;
  if (threadIdx.x == 0) s_skip = (*(volatile int32_t*)dev_err != 0) ? 1 : 0;
  __syncthreads();
  if (s_skip) return;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  const int num_kb = (K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(ready_bar(s), 4);
      mbar_init(empty_bar(s), 1);
    }
    mbar_init(tmem_full_bar, 1);
    mbar_init(tmem_empty_bar, 4);
    *s_abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    fence_proxy_async();
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32((const void*)s_tmem)),
                 "r"((uint32_t)BN)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *s_tmem;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer ---
    if (lane == 0) {
      for (int kb = 0; kb < num_kb; ++kb) {
        const int s = kb % STAGES;
        const uint32_t ph = (uint32_t)(kb / STAGES) & 1u;
        if (!mbar_wait(empty_bar(s), ph ^ 1u, s_abort)) break;
        mbar_arrive_expect_tx(full_bar(s), (uint32_t)(cfg::A_BYTES + cfg::B_BYTES));
        const uint32_t a_dst = smem_base + (uint32_t)(s * cfg::STAGE_BYTES);
        const uint32_t b_dst = a_dst + (uint32_t)((PASSES == 3 ? 2 : 1) * cfg::A_BYTES);
        const int k0 = kb * BK;
        if (A_MN) {
#pragma unroll
          for (int c = 0; c < BM / 32; ++c) tma_load_2d(a_dst + (uint32_t)(c * BK * 128), &tmA, m0 + 32 * c, k0, full_bar(s));
        } else {
          tma_load_2d(a_dst, &tmA, k0, m0, full_bar(s));
        }
        if (B_MN) {
#pragma unroll
          for (int c = 0; c < BN / 32; ++c) tma_load_2d(b_dst + (uint32_t)(c * BK * 128), &tmB, n0 + 32 * c, k0, full_bar(s));
        } else {
          tma_load_2d(b_dst, &tmB, k0, n0, full_bar(s));
        }
      }
    }
  } else if (warp == 1) {
    // -------------------------------------------------------------------- MMA issuer ---
    if (lane == 0) {
      // instruction descriptor: D = F32, A = B = TF32, majors, N >> 3, M >> 4
      const uint32_t idesc = (1u << 4) | (2u << 7) | (2u << 10) | ((A_MN ? 1u : 0u) << 15) | ((B_MN ? 1u : 0u) << 16) |
                             ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
      bool ok = true;
      for (int kb = 0; kb < num_kb && ok; ++kb) {
        const int s = kb % STAGES;
        const uint32_t ph = (uint32_t)(kb / STAGES) & 1u;
        const int seg = kb / SEG_KB, kb_in_seg = kb % SEG_KB;
        if (kb_in_seg == 0 && seg > 0) {
          // the epilogue warps must have drained the previous segment out of tensor memory
          ok = mbar_wait(tmem_empty_bar, (uint32_t)(seg - 1) & 1u, s_abort);
          if (!ok) break;
        }
        ok = mbar_wait(PASSES == 3 ? ready_bar(s) : full_bar(s), ph, s_abort);
        if (!ok) break;
        tc_fence_after();
        const uint32_t a_hi = smem_base + (uint32_t)(s * cfg::STAGE_BYTES);
        const uint32_t a_lo = a_hi + (uint32_t)cfg::A_BYTES;
        const uint32_t b_hi = a_hi + (uint32_t)((PASSES == 3 ? 2 : 1) * cfg::A_BYTES);
        const uint32_t b_lo = b_hi + (uint32_t)cfg::B_BYTES;
#pragma unroll
        for (int kk = 0; kk < BK / 8; ++kk) {
          // one MMA covers 8 k-values: 32 bytes along a K-major row, eight 128-byte k-rows of an MN-major tile
          const uint32_t a_off = A_MN ? (uint32_t)(kk * 1024) : (uint32_t)(kk * 32);
          const uint32_t b_off = B_MN ? (uint32_t)(kk * 1024) : (uint32_t)(kk * 32);
          const uint64_t da_hi = A_MN ? make_smem_desc(a_hi + a_off, BK * 128, 512, LAYOUT_SW128_32B)
                                      : make_smem_desc(a_hi + a_off, 16, 512, LAYOUT_SW64);
          const uint64_t db_hi = B_MN ? make_smem_desc(b_hi + b_off, BK * 128, 512, LAYOUT_SW128_32B)
                                      : make_smem_desc(b_hi + b_off, 16, 512, LAYOUT_SW64);
          const uint32_t first = (kb_in_seg > 0 || kk > 0) ? 1u : 0u;
          if (PASSES == 3) {
            const uint64_t da_lo = A_MN ? make_smem_desc(a_lo + a_off, BK * 128, 512, LAYOUT_SW128_32B)
                                        : make_smem_desc(a_lo + a_off, 16, 512, LAYOUT_SW64);
            const uint64_t db_lo = B_MN ? make_smem_desc(b_lo + b_off, BK * 128, 512, LAYOUT_SW128_32B)
                                        : make_smem_desc(b_lo + b_off, 16, 512, LAYOUT_SW64);
            tc_mma_tf32(tmem_base, da_lo, db_hi, idesc, first);
            tc_mma_tf32(tmem_base, da_hi, db_lo, idesc, 1u);
            tc_mma_tf32(tmem_base, da_hi, db_hi, idesc, 1u);
          } else {
            tc_mma_tf32(tmem_base, da_hi, db_hi, idesc, first);
          }
        }
        tc_commit(empty_bar(s));   // frees the stage once these MMAs have read it
        if (kb_in_seg == SEG_KB - 1 || kb == num_kb - 1) tc_commit(tmem_full_bar);   // segment complete
      }
    }
  } else {
    // ------------------------------------- hi / lo split, and the epilogue per K segment ---
    const int tt = threadIdx.x - 64;  // 0..127
    const int q = warp & 3;           // TMEM lane quadrant this warp may read
    const int row = m0 + 32 * q + lane;
    float* crow = C + (int64_t)row * ldc;
    float* zrow = Z ? Z + (int64_t)row * ldc : nullptr;
    const int num_seg = (num_kb + SEG_KB - 1) / SEG_KB;
    bool ok = true;

    // Drains the accumulator of segment `seg`: intermediate segments add into C (round-to-nearest fp32 adds),
    // the last one also applies bias, pre-activation store and activation.
    auto drain = [&](int seg) -> bool {
      if (!mbar_wait(tmem_full_bar, (uint32_t)seg & 1u, s_abort)) return false;
      tc_fence_after();
      const bool last = (seg == num_seg - 1);
      const bool add_c = (seg > 0) || (accumulate != 0);
#pragma unroll 1
      for (int cc = 0; cc < BN / 32; ++cc) {
        const int nb = n0 + cc * 32;
        if (nb >= N) break;   // warp-uniform
        uint32_t r[32];
        tc_ld_32x32b_x32(tmem_base + ((uint32_t)(32 * q) << 16) + (uint32_t)(cc * 32), r);
        tc_wait_ld();
        if (row < M) {
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const int n = nb + 4 * j;
            float v[4] = {__uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1]), __uint_as_float(r[4 * j + 2]),
                          __uint_as_float(r[4 * j + 3])};
            if (n + 3 < N) {
              if (add_c) {
                const float4 c4 = *(const float4*)(crow + n);
                v[0] += c4.x; v[1] += c4.y; v[2] += c4.z; v[3] += c4.w;
              }
              if (last) {
                if (bias_n) {
                  const float4 b4 = __ldg((const float4*)(bias_n + n));
                  v[0] += b4.x; v[1] += b4.y; v[2] += b4.z; v[3] += b4.w;
                }
                if (zrow) *(float4*)(zrow + n) = make_float4(v[0], v[1], v[2], v[3]);
                if (act != FB_ACT_IDENTITY) {
#pragma unroll
                  for (int e = 0; e < 4; ++e) v[e] = fb_act_apply(act, v[e]);
                }
              }
              *(float4*)(crow + n) = make_float4(v[0], v[1], v[2], v[3]);
            } else {
              for (int e = 0; e < 4 && n + e < N; ++e) {
                float u = v[e];
                if (add_c) u += crow[n + e];
                if (last) {
                  if (bias_n) u += __ldg(bias_n + n + e);
                  if (zrow) zrow[n + e] = u;
                  u = fb_act_apply(act, u);
                }
                crow[n + e] = u;
              }
            }
          }
        }
      }
      if (!last) {
        // tensor memory may be overwritten by the next segment once every warp has read its quadrant
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(tmem_empty_bar);
      }
      return true;
    };

    if (PASSES == 3) {
      for (int kb = 0; kb < num_kb && ok; ++kb) {
        const int s = kb % STAGES;
        const uint32_t ph = (uint32_t)(kb / STAGES) & 1u;
        ok = mbar_wait(full_bar(s), ph, s_abort);
        if (!ok) break;
        float4* a_hi = (float4*)(smem + s * cfg::STAGE_BYTES);
        float4* a_lo = (float4*)(smem + s * cfg::STAGE_BYTES + cfg::A_BYTES);
        float4* b_hi = (float4*)(smem + s * cfg::STAGE_BYTES + 2 * cfg::A_BYTES);
        float4* b_lo = (float4*)(smem + s * cfg::STAGE_BYTES + 2 * cfg::A_BYTES + cfg::B_BYTES);
#pragma unroll
        for (int i = 0; i < cfg::A_BYTES / 16 / 128; ++i) {
          const float4 v = a_hi[tt + i * 128];
          float4 h, l;
          h.x = __uint_as_float(__float_as_uint(v.x) & 0xffffe000u); l.x = v.x - h.x;
          h.y = __uint_as_float(__float_as_uint(v.y) & 0xffffe000u); l.y = v.y - h.y;
          h.z = __uint_as_float(__float_as_uint(v.z) & 0xffffe000u); l.z = v.z - h.z;
          h.w = __uint_as_float(__float_as_uint(v.w) & 0xffffe000u); l.w = v.w - h.w;
          a_hi[tt + i * 128] = h;
          a_lo[tt + i * 128] = l;
        }
#pragma unroll
        for (int i = 0; i < cfg::B_BYTES / 16 / 128; ++i) {
          const float4 v = b_hi[tt + i * 128];
          float4 h, l;
          h.x = __uint_as_float(__float_as_uint(v.x) & 0xffffe000u); l.x = v.x - h.x;
          h.y = __uint_as_float(__float_as_uint(v.y) & 0xffffe000u); l.y = v.y - h.y;
          h.z = __uint_as_float(__float_as_uint(v.z) & 0xffffe000u); l.z = v.z - h.z;
          h.w = __uint_as_float(__float_as_uint(v.w) & 0xffffe000u); l.w = v.w - h.w;
          b_hi[tt + i * 128] = h;
          b_lo[tt + i * 128] = l;
        }
        fence_proxy_async();   // generic-proxy writes become visible to the tensor core's async-proxy reads
        __syncwarp();
        if (lane == 0) mbar_arrive(ready_bar(s));
        if (kb % SEG_KB == SEG_KB - 1 || kb == num_kb - 1) ok = drain(kb / SEG_KB);
      }
    } else {
      for (int seg = 0; seg < num_seg && ok; ++seg) ok = drain(seg);
    }
  }

  // ---------------------------------------------------------------------- teardown ---
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)BN) : "memory");
  }
  if (threadIdx.x == 0 && *s_abort != 0) atomicExch(dev_err, 1001);
}

// --------------------------------------------------------------------------- host side ---
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = (EncodeTiledFn)p;
    else
      cudaGetLastError();
  }
  return fn;
}

// 2-D fp32 tensor map over a row-major [rows][cols] matrix with leading dimension ld (floats).
bool encode_map(CUtensorMap* map, const float* base, int64_t rows, int64_t cols, int64_t ld, uint32_t box_cols,
                uint32_t box_rows, CUtensorMapSwizzle swz) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return false;
  cuuint64_t gdim[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t gstride[1] = {(cuuint64_t)ld * sizeof(float)};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, (void*)base, gdim, gstride, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, swz, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

template <bool A_MN, bool B_MN, int BN, int PASSES>
int32_t launch_variant(fb_ctx* ctx, cudaStream_t stream, const fb_gemm_args& a) {
  using cfg = Cfg<BN, PASSES>;
  CUtensorMap tmA, tmB;
  bool ok;
  if (A_MN) ok = encode_map(&tmA, a.A, a.K, a.M, a.lda, 32, BK, CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B);
  else ok = encode_map(&tmA, a.A, a.M, a.K, a.lda, BK, BM, CU_TENSOR_MAP_SWIZZLE_64B);
  if (ok) {
    if (B_MN) ok = encode_map(&tmB, a.B, a.K, a.N, a.ldb, 32, BK, CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B);
    else ok = encode_map(&tmB, a.B, a.N, a.K, a.ldb, BK, BN, CU_TENSOR_MAP_SWIZZLE_64B);
  }
  if (!ok) return fb_fail(FB_ERR_CUDA, "gemm: cuTensorMapEncodeTiled failed (M=%lld N=%lld K=%lld lda=%lld ldb=%lld)",
                          (long long)a.M, (long long)a.N, (long long)a.K, (long long)a.lda, (long long)a.ldb);
  auto kern = gemm_tc_kernel<A_MN, B_MN, BN, PASSES>;
  static bool attr_set = false;
  if (!attr_set) {
    FB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, cfg::SMEM_BYTES));
    attr_set = true;
  }
  dim3 grid((unsigned)((a.N + BN - 1) / BN), (unsigned)((a.M + BM - 1) / BM));
  kern<<<grid, NUM_THREADS, cfg::SMEM_BYTES, stream>>>(tmA, tmB, a.C, a.ldc, a.Z, a.bias_n, (int)a.M, (int)a.N, (int)a.K,
                                                       a.act, a.accumulate, ctx->dev_error);
  FB_LAUNCH_CHECK();
  return FB_OK;
}

template <int BN, int PASSES>
int32_t launch_layout(fb_ctx* ctx, cudaStream_t stream, const fb_gemm_args& a) {
  if (a.a_mn_major) {
    if (a.b_mn_major) return launch_variant<true, true, BN, PASSES>(ctx, stream, a);
    return launch_variant<true, false, BN, PASSES>(ctx, stream, a);
  }
  if (a.b_mn_major) return launch_variant<false, true, BN, PASSES>(ctx, stream, a);
  return launch_variant<false, false, BN, PASSES>(ctx, stream, a);
}

}  // namespace

bool fb_gemm_tc_supported(const fb_gemm_args& a) {
  if (a.M < 1 || a.N < 1 || a.K < 1) return false;
  if (a.M > 0x7fffff00 || a.N > 0x7fffff00 || a.K > 0x7fffff00) return false;
  if ((a.M + BM - 1) / BM > 65535) return false;
  if (a.bias_m != nullptr) return false;
  if (!fb_aligned16(a.A) || !fb_aligned16(a.B) || !fb_aligned16(a.C)) return false;
  if (a.Z && !fb_aligned16(a.Z)) return false;
  if (a.bias_n && !fb_aligned16(a.bias_n)) return false;
  if (a.lda % 4 || a.ldb % 4 || a.ldc % 4) return false;
  // the leading dimension must cover the contiguous extent
  if (a.lda < (a.a_mn_major ? a.M : a.K) || a.ldb < (a.b_mn_major ? a.N : a.K) || a.ldc < a.N) return false;
  return true;
}

int32_t fb_gemm_tc_launch(fb_ctx* ctx, cudaStream_t stream, const fb_gemm_args& a, int passes) {
  if (!fb_gemm_tc_supported(a)) return FB_ERR_UNSUPPORTED;
  const int64_t tiles256 = ((a.M + BM - 1) / BM) * ((a.N + 255) / 256);
  const bool narrow = (a.N <= 128) || (tiles256 < ctx->sm_count);
  if (passes == 3) {
    if (narrow) return launch_layout<128, 3>(ctx, stream, a);
    return launch_layout<256, 3>(ctx, stream, a);
  }
  if (narrow) return launch_layout<128, 1>(ctx, stream, a);
  return launch_layout<256, 1>(ctx, stream, a);
}

void fb_tmap_cache_destroy(fb_ctx* ctx) { (void)ctx; }
