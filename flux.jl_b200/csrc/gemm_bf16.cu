// Tensor-core GEMM for BFloat16 data on sm_100a (the opt-in bf16 path of Flux.bf16): TMA -> shared memory ->
// tcgen05.mma.kind::f16 with bf16 operands and fp32 accumulators in tensor memory -> tcgen05.ld epilogue with fused
// bias / activation / pre-activation store, results written as bf16 (or fp32).
//
// Compared with the Float32 kernel (3xTF32) there is one MMA pass, no operand splitting and half the bytes per
// element, so a k-block is 64 values (128 bytes) and the ring holds 4-6 stages of 32-48 KB.
//
// Tiles.  A cluster of two CTAs computes a 256 x 256 tile of row-major C[M][N] with cta_group::2 MMAs (each CTA loads
// 128 rows of A and 128 columns of B; the leader issues one M = 256, N = 256, K = 16 MMA per 32 bytes of k); small
// problems use one CTA per 128 x 128 tile.  The kernel is persistent: CTA (pair) c of G walks tiles c, c + G, ...; the
// stage ring and the two accumulator buffers in tensor memory run on across tiles, so the epilogue of one tile
// overlaps the main loop of the next.
//
// Warp roles: warp 0 issues the TMA loads, warp 1 owns tensor memory and issues the MMAs, warps 2-5 are the
// epilogue (one TMEM lane quadrant each).  In a pair the leader's MMA reads both CTAs' shared memory, so both CTAs'
// loads (cta_group::2 form) complete on the LEADER's full barrier, which expects the bytes of both halves.
//
// Operand layouts in shared memory are the canonical 128-byte-swizzle layouts the MMA descriptors name: K-major
// tiles are rows of 128 bytes in 8-row atoms (SBO = 1024); MN-major tiles are chunks of 64 MN-values x BK k-rows of
// 128 bytes (LBO = chunk stride, SBO = 1024 for 8 k-rows).  No TMA load is multicast.  Every mbarrier wait is
// bounded; when one runs out the kernel records code 1101 / 1102 in the device error word and returns.
#include <cuda.h>
#include <cuda_bf16.h>
#include <stdlib.h>

#include "common.cuh"
#include "tc_common.cuh"

namespace {

constexpr int HBM_ = 128;            // rows of A per CTA
constexpr int HBK = 64;              // bf16 values per k-block (128 bytes)
constexpr uint32_t LAYOUT_SW128 = 2;

template <int BN, bool PAIR>
struct HCfg {
  static constexpr int BNC = PAIR ? BN / 2 : BN;              // B columns this CTA loads per stage
  static constexpr int A_BYTES = HBM_ * HBK * 2;              // 16 KB
  static constexpr int B_BYTES = BNC * HBK * 2;               // 16 KB at 128 columns
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGES = (196608 / STAGE_BYTES) > 8 ? 8 : (196608 / STAGE_BYTES);
  static constexpr int BAR_OFFSET = STAGES * STAGE_BYTES;
  static constexpr int SMEM_BYTES = BAR_OFFSET + 512 + 1024;  // barriers + alignment slack
  static constexpr int TMEM_COLS = 2 * BN;                    // two accumulator buffers
  static constexpr int NUM_THREADS = 32 * 6;
  static constexpr uint32_t ARRIVALS = PAIR ? 8 : 4;          // epilogue warps arriving on tmem_empty
};

__device__ __forceinline__ void tc_mma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %6, %7, %8}, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(0u), "r"(0u), "r"(0u), "r"(0u)
      : "memory");
}
__device__ __forceinline__ void tc_mma2_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, {%5, %6, %7, %8, %9, %10, %11, %12}, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(0u), "r"(0u), "r"(0u), "r"(0u), "r"(0u),
      "r"(0u), "r"(0u), "r"(0u)
      : "memory");
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&v);
}
__device__ __forceinline__ float bf16_lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t w) { return __uint_as_float(w & 0xffff0000u); }

template <bool A_MN, bool B_MN, int BN, bool PAIR>
__global__ void __launch_bounds__(HCfg<BN, PAIR>::NUM_THREADS, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, void* __restrict__ Cv,
                 int64_t ldc, uint16_t* __restrict__ Z, const uint16_t* __restrict__ bias_n, int M, int N, int K, int act,
                 int accumulate, int out_f32, int32_t* __restrict__ dev_err, int a3d, int b3d, int num_tiles, int tiles_n) {
  using cfg = HCfg<BN, PAIR>;
  constexpr int STAGES = cfg::STAGES;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const uint32_t smem_base = smem_u32(smem);
  uint64_t* bars = (uint64_t*)(smem + cfg::BAR_OFFSET);
  const uint32_t bar_base = smem_base + cfg::BAR_OFFSET;
  // barrier slots: full[S], empty[S], (unused)[S], tmem_full[2], tmem_empty[2]
  auto full_bar = [&](int s) { return bar_base + 8u * (uint32_t)s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (uint32_t)(STAGES + s); };
  auto tmem_full_bar = [&](int b) { return bar_base + 8u * (uint32_t)(3 * STAGES + b); };
  auto tmem_empty_bar = [&](int b) { return bar_base + 8u * (uint32_t)(3 * STAGES + 2 + b); };
  volatile uint32_t* s_tmem = (volatile uint32_t*)(bars + 3 * STAGES + 4);
  volatile int* s_abort = (volatile int*)(bars + 3 * STAGES + 5);
  volatile int* s_skip = (volatile int*)(bars + 3 * STAGES + 6);   // [0] mine, [1] written by the peer CTA

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = PAIR ? cluster_ctarank() : 0u;
  const bool leader = (rank == 0);
  const int cid = PAIR ? (int)(blockIdx.x >> 1) : (int)blockIdx.x;
  const int G = PAIR ? (int)(gridDim.x >> 1) : (int)gridDim.x;
  const int num_kb = (K + HBK - 1) / HBK;
  auto tile_m0 = [&](int t) { return PAIR ? (t / tiles_n) * 256 + 128 * (int)rank : (t / tiles_n) * HBM_; };
  auto tile_n0 = [&](int t) { return (t % tiles_n) * BN; };

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(tmem_full_bar(b), 1);
      mbar_init(tmem_empty_bar(b), cfg::ARRIVALS);
    }
    *s_abort = 0;
    s_skip[0] = (*(volatile int32_t*)dev_err != 0) ? 1 : 0;   // an error word left set means: do not start
    s_skip[1] = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    fence_proxy_async();
  }
  if (PAIR) {
    __syncwarp();
    cluster_sync_all();   // both CTAs run and their barriers exist: remote accesses may start
    if (threadIdx.x == 0) {
      asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(map_to_cta(smem_u32((const void*)(s_skip + 1)), rank ^ 1u)),
                   "r"((int)s_skip[0])
                   : "memory");
    }
    __syncwarp();
    cluster_sync_all();
  } else {
    __syncthreads();
  }
  if (s_skip[0] != 0 || s_skip[1] != 0) return;   // uniform over the CTA (pair)

  if (warp == 1) {
    if (PAIR) {
      asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32((const void*)s_tmem)),
                   "r"((uint32_t)cfg::TMEM_COLS)
                   : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    } else {
      asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32((const void*)s_tmem)),
                   "r"((uint32_t)cfg::TMEM_COLS)
                   : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *s_tmem;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer ---
    if (lane == 0) {
      int it = 0;   // k-blocks issued so far over all tiles: names the stage and its phase
      bool ok = true;
      for (int t = cid; t < num_tiles && ok; t += G) {
        const int m0 = tile_m0(t);
        const int nb0 = tile_n0(t) + (PAIR ? cfg::BNC * (int)rank : 0);
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (uint32_t)(it / STAGES) & 1u;
          ok = mbar_wait_cluster(empty_bar(s), ph ^ 1u, s_abort);
          if (!ok) break;
          // pairs: the leader's barrier counts the bytes of both CTAs' halves; the peer only issues its loads
          const uint32_t fb = PAIR ? map_to_cta(full_bar(s), 0u) : full_bar(s);
          if (!PAIR || leader) mbar_arrive_expect_tx(full_bar(s), (uint32_t)((PAIR ? 2 : 1) * (cfg::A_BYTES + cfg::B_BYTES)));
          const uint32_t a_dst = smem_base + (uint32_t)(s * cfg::STAGE_BYTES);
          const uint32_t b_dst = a_dst + (uint32_t)cfg::A_BYTES;
          const int k0 = kb * HBK;
          auto load2 = [&](uint32_t dst, const CUtensorMap* map, int x, int y) {
            if (PAIR) tma_load_2d_pair(dst, map, x, y, fb);
            else tma_load_2d(dst, map, x, y, fb);
          };
          auto load3 = [&](uint32_t dst, const CUtensorMap* map, int x, int y, int z) {
            if (PAIR) tma_load_3d_pair(dst, map, x, y, z, fb);
            else tma_load_3d(dst, map, x, y, z, fb);
          };
          if (A_MN) {
            if (a3d) {
              load3(a_dst, &tmA, 0, k0, m0 >> 6);
            } else {
#pragma unroll
              for (int c = 0; c < HBM_ / 64; ++c) load2(a_dst + (uint32_t)(c * HBK * 128), &tmA, m0 + 64 * c, k0);
            }
          } else {
            load2(a_dst, &tmA, k0, m0);
          }
          if (B_MN) {
            if (b3d) {
              load3(b_dst, &tmB, 0, k0, nb0 >> 6);
            } else {
#pragma unroll
              for (int c = 0; c < cfg::BNC / 64; ++c) load2(b_dst + (uint32_t)(c * HBK * 128), &tmB, nb0 + 64 * c, k0);
            }
          } else {
            load2(b_dst, &tmB, k0, nb0);
          }
        }
      }
    }
  } else if (warp == 1) {
    // -------------------------------------------------- MMA issuer (the leader CTA of a pair) ---
    if (lane == 0 && leader) {
      // instruction descriptor: D = F32, A = B = BF16, operand majors, N >> 3, M >> 4
      const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((A_MN ? 1u : 0u) << 15) | ((B_MN ? 1u : 0u) << 16) |
                             ((uint32_t)(BN >> 3) << 17) | ((uint32_t)((PAIR ? 256 : HBM_) >> 4) << 24);
      bool ok = true;
      int it = 0, tc = 0;   // k-blocks and tiles issued so far
      for (int t = cid; t < num_tiles && ok; t += G, ++tc) {
        const int buf = tc & 1, use = tc >> 1;
        if (use > 0) {
          // the epilogue warps must have drained this accumulator buffer's previous tile
          ok = mbar_wait_cluster(tmem_empty_bar(buf), (uint32_t)(use - 1) & 1u, s_abort);
          if (!ok) break;
        }
        const uint32_t d_tmem = tmem_base + (uint32_t)(buf * BN);
        for (int kb = 0; kb < num_kb && ok; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (uint32_t)(it / STAGES) & 1u;
          ok = mbar_wait_cluster(full_bar(s), ph, s_abort);
          if (!ok) break;
          tc_fence_after();
          const uint32_t a_s = smem_base + (uint32_t)(s * cfg::STAGE_BYTES);
          const uint32_t b_s = a_s + (uint32_t)cfg::A_BYTES;
#pragma unroll
          for (int kk = 0; kk < HBK / 16; ++kk) {
            // one MMA covers 16 k-values: 32 bytes along a K-major row, sixteen 128-byte k-rows of an MN-major tile
            const uint32_t a_off = A_MN ? (uint32_t)(kk * 2048) : (uint32_t)(kk * 32);
            const uint32_t b_off = B_MN ? (uint32_t)(kk * 2048) : (uint32_t)(kk * 32);
            const uint64_t da = A_MN ? make_smem_desc(a_s + a_off, HBK * 128, 1024, LAYOUT_SW128)
                                     : make_smem_desc(a_s + a_off, 16, 1024, LAYOUT_SW128);
            const uint64_t db = B_MN ? make_smem_desc(b_s + b_off, HBK * 128, 1024, LAYOUT_SW128)
                                     : make_smem_desc(b_s + b_off, 16, 1024, LAYOUT_SW128);
            const uint32_t acc = (kb > 0 || kk > 0) ? 1u : 0u;
            if (PAIR) tc_mma2_f16(d_tmem, da, db, idesc, acc);
            else tc_mma_f16(d_tmem, da, db, idesc, acc);
          }
          const bool last = (kb == num_kb - 1);
          if (PAIR) {
            tc_commit2_mc(empty_bar(s), (uint16_t)3);                 // frees the stage in both CTAs
            if (last) tc_commit2_mc(tmem_full_bar(buf), (uint16_t)3);
          } else {
            tc_commit(empty_bar(s));
            if (last) tc_commit(tmem_full_bar(buf));
          }
        }
      }
    }
  } else {
    // -------------------------------------------------------------- epilogue warps ---
    const int q = warp & 3;                 // TMEM lane quadrant this warp may read
    bool ok = true;
    int tc = 0;
    for (int t = cid; t < num_tiles && ok; t += G, ++tc) {
      const int buf = tc & 1, use = tc >> 1;
      const int n0 = tile_n0(t);
      const int row = tile_m0(t) + 32 * q + lane;
      ok = mbar_wait_cluster(tmem_full_bar(buf), (uint32_t)use & 1u, s_abort);
      if (!ok) break;
      tc_fence_after();
#pragma unroll 1
      for (int cc = 0; cc < BN / 32; ++cc) {
        const int nb = n0 + cc * 32;
        if (nb >= N) break;   // warp-uniform
        uint32_t r[32];
        tc_ld_32x32b_x32(tmem_base + ((uint32_t)(32 * q) << 16) + (uint32_t)(buf * BN + cc * 32), r);
        tc_wait_ld();
        float* v = reinterpret_cast<float*>(r);
        if (row < M) {
          const bool full = (nb + 31 < N);
          if (out_f32) {
            float* crow = (float*)Cv + (int64_t)row * ldc + nb;
            for (int e = 0; e < 32 && nb + e < N; ++e) {
              float x = v[e];
              if (accumulate) x += crow[e];
              if (bias_n) x += bf16_lo((uint32_t)bias_n[nb + e]);
              if (Z) Z[(int64_t)row * ldc + nb + e] = (uint16_t)(pack_bf16(x, 0.0f) & 0xffffu);
              crow[e] = fb_act_apply(act, x);
            }
          } else if (full) {
            uint16_t* crow = (uint16_t*)Cv + (int64_t)row * ldc + nb;
            uint16_t* zrow = Z ? Z + (int64_t)row * ldc + nb : nullptr;
#pragma unroll
            for (int j = 0; j < 4; ++j) {       // 8 columns = one 16-byte store
              float u[8];
#pragma unroll
              for (int e = 0; e < 8; ++e) u[e] = v[8 * j + e];
              if (accumulate) {
                const uint4 c4 = *(const uint4*)(crow + 8 * j);
                u[0] += bf16_lo(c4.x); u[1] += bf16_hi(c4.x); u[2] += bf16_lo(c4.y); u[3] += bf16_hi(c4.y);
                u[4] += bf16_lo(c4.z); u[5] += bf16_hi(c4.z); u[6] += bf16_lo(c4.w); u[7] += bf16_hi(c4.w);
              }
              if (bias_n) {
                const uint4 b4 = __ldg((const uint4*)(bias_n + nb + 8 * j));
                u[0] += bf16_lo(b4.x); u[1] += bf16_hi(b4.x); u[2] += bf16_lo(b4.y); u[3] += bf16_hi(b4.y);
                u[4] += bf16_lo(b4.z); u[5] += bf16_hi(b4.z); u[6] += bf16_lo(b4.w); u[7] += bf16_hi(b4.w);
              }
              if (zrow) *(uint4*)(zrow + 8 * j) = make_uint4(pack_bf16(u[0], u[1]), pack_bf16(u[2], u[3]), pack_bf16(u[4], u[5]), pack_bf16(u[6], u[7]));
              if (act != FB_ACT_IDENTITY) {
#pragma unroll
                for (int e = 0; e < 8; ++e) u[e] = fb_act_apply(act, u[e]);
              }
              *(uint4*)(crow + 8 * j) = make_uint4(pack_bf16(u[0], u[1]), pack_bf16(u[2], u[3]), pack_bf16(u[4], u[5]), pack_bf16(u[6], u[7]));
            }
          } else {
            uint16_t* crow = (uint16_t*)Cv + (int64_t)row * ldc + nb;
            for (int e = 0; e < 32 && nb + e < N; ++e) {
              float x = v[e];
              if (accumulate) x += bf16_lo((uint32_t)crow[e]);
              if (bias_n) x += bf16_lo((uint32_t)bias_n[nb + e]);
              if (Z) Z[(int64_t)row * ldc + nb + e] = (uint16_t)(pack_bf16(x, 0.0f) & 0xffffu);
              crow[e] = (uint16_t)(pack_bf16(fb_act_apply(act, x), 0.0f) & 0xffffu);
            }
          }
        }
      }
      // this buffer may be overwritten once every epilogue warp (of both CTAs) has read its quadrant
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        if (PAIR) mbar_arrive_cluster(map_to_cta(tmem_empty_bar(buf), 0u));
        else mbar_arrive(tmem_empty_bar(buf));
      }
    }
  }

  // ---------------------------------------------------------------------- teardown ---
  tc_fence_before();
  __syncthreads();
  if (PAIR) cluster_sync_all();   // neither CTA may release tensor memory while its peer can still touch it
  if (warp == 1) {
    __syncwarp();
    if (PAIR)
      asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)cfg::TMEM_COLS) : "memory");
    else
      asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)cfg::TMEM_COLS) : "memory");
  }
  if (threadIdx.x == 0 && *s_abort != 0) atomicExch(dev_err, PAIR ? 1102 : 1101);
}

// --------------------------------------------------------------------------- host side ---
// 2-D bf16 tensor map over a row-major [rows][cols] matrix with leading dimension ld (elements).
bool encode_map_bf16(CUtensorMap* map, const uint16_t* base, int64_t rows, int64_t cols, int64_t ld, uint32_t box_cols,
                     uint32_t box_rows) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return false;
  cuuint64_t gdim[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t gstride[1] = {(cuuint64_t)ld * 2};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (void*)base, gdim, gstride, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
            CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// 3-d view {64, K, MN / 64} of an MN-major matrix (row k holds MN contiguous values): box {64, HBK, chunks}.
bool encode_map_bf16_mn3d(CUtensorMap* map, const uint16_t* base, int64_t K, int64_t MN, int64_t ld, uint32_t chunks) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn || MN % 64 != 0) return false;
  cuuint64_t gdim[3] = {64, (cuuint64_t)K, (cuuint64_t)(MN / 64)};
  cuuint64_t gstride[2] = {(cuuint64_t)ld * 2, 128};
  cuuint32_t box[3] = {64, (cuuint32_t)HBK, chunks};
  cuuint32_t estr[3] = {1, 1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, (void*)base, gdim, gstride, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
            CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <bool A_MN, bool B_MN, int BN, bool PAIR>
int32_t launch_bf16(fb_ctx* ctx, cudaStream_t stream, const fb_gemm_bf16_args& a) {
  using cfg = HCfg<BN, PAIR>;
  CUtensorMap tmA, tmB;
  bool ok;
  int a3d = 0, b3d = 0;
  if (A_MN) {
    a3d = encode_map_bf16_mn3d(&tmA, a.A, a.K, a.M, a.lda, HBM_ / 64) ? 1 : 0;
    ok = a3d || encode_map_bf16(&tmA, a.A, a.K, a.M, a.lda, 64, HBK);
  } else {
    ok = encode_map_bf16(&tmA, a.A, a.M, a.K, a.lda, HBK, HBM_);
  }
  if (ok) {
    if (B_MN) {
      b3d = encode_map_bf16_mn3d(&tmB, a.B, a.K, a.N, a.ldb, cfg::BNC / 64) ? 1 : 0;
      ok = b3d || encode_map_bf16(&tmB, a.B, a.K, a.N, a.ldb, 64, HBK);
    } else {
      ok = encode_map_bf16(&tmB, a.B, a.N, a.K, a.ldb, HBK, cfg::BNC);
    }
  }
  if (!ok) return fb_fail(FB_ERR_CUDA, "bf16 gemm: cuTensorMapEncodeTiled failed (M=%lld N=%lld K=%lld lda=%lld ldb=%lld)",
                          (long long)a.M, (long long)a.N, (long long)a.K, (long long)a.lda, (long long)a.ldb);
  auto kern = gemm_bf16_kernel<A_MN, B_MN, BN, PAIR>;
  FB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, cfg::SMEM_BYTES));
  // the whole L1 / shared array as shared memory: the communication-stream kernels ask for the same split, and an SM
  // takes CTAs of two kernels together only when their splits agree
  FB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared));
  const int tiles_n = (int)((a.N + BN - 1) / BN);
  const int64_t tiles_m = PAIR ? (a.M + 255) / 256 : (a.M + HBM_ - 1) / HBM_;
  const int64_t num_tiles = tiles_m * tiles_n;
  if (num_tiles > 0x7fffffff) return fb_fail(FB_ERR_UNSUPPORTED, "bf16 gemm: too many tiles");
  const int sms = ctx->sm_count - ctx->reserved_sms;
  const int64_t Gmax = PAIR ? (sms / 2 > 0 ? sms / 2 : 1) : sms;
  const int64_t G = Gmax < num_tiles ? Gmax : num_tiles;
  cudaLaunchConfig_t lc;
  memset(&lc, 0, sizeof(lc));
  lc.gridDim = dim3((unsigned)(PAIR ? 2 * G : G), 1, 1);
  lc.blockDim = dim3(cfg::NUM_THREADS, 1, 1);
  lc.dynamicSmemBytes = cfg::SMEM_BYTES;
  lc.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = PAIR ? 2 : 1;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  lc.attrs = attr;
  lc.numAttrs = 1;
  FB_CUDA(cudaLaunchKernelEx(&lc, kern, tmA, tmB, a.C, a.ldc, a.Z, a.bias_n, (int)a.M, (int)a.N, (int)a.K, a.act, a.accumulate,
                             a.out_f32, ctx->dev_error, a3d, b3d, (int)num_tiles, tiles_n));
  FB_LAUNCH_CHECK();
  return FB_OK;
}

template <int BN, bool PAIR>
int32_t launch_bf16_layout(fb_ctx* ctx, cudaStream_t stream, const fb_gemm_bf16_args& a) {
  if (a.a_mn_major) {
    if (a.b_mn_major) return launch_bf16<true, true, BN, PAIR>(ctx, stream, a);
    return launch_bf16<true, false, BN, PAIR>(ctx, stream, a);
  }
  if (a.b_mn_major) return launch_bf16<false, true, BN, PAIR>(ctx, stream, a);
  return launch_bf16<false, false, BN, PAIR>(ctx, stream, a);
}

}  // namespace

bool fb_gemm_bf16_supported(const fb_gemm_bf16_args& a) {
  if (a.M < 1 || a.N < 1 || a.K < 1) return false;
  if (a.M > 0x7fffff00 || a.N > 0x7fffff00 || a.K > 0x7fffff00) return false;
  if (!fb_aligned16(a.A) || !fb_aligned16(a.B) || !fb_aligned16(a.C)) return false;
  if (a.Z && !fb_aligned16(a.Z)) return false;
  if (a.bias_n && !fb_aligned16(a.bias_n)) return false;
  if (a.lda % 8 || a.ldb % 8) return false;                       // TMA strides are multiples of 16 bytes
  if (a.ldc % (a.out_f32 ? 4 : 8)) return false;
  if (a.lda < (a.a_mn_major ? a.M : a.K) || a.ldb < (a.b_mn_major ? a.N : a.K) || a.ldc < a.N) return false;
  return true;
}

int32_t fb_gemm_bf16_launch(fb_ctx* ctx, cudaStream_t stream, const fb_gemm_bf16_args& a) {
  if (!fb_gemm_bf16_supported(a))
    return fb_fail(FB_ERR_UNSUPPORTED,
                   "bf16 gemm: needs 16-byte aligned pointers and leading dimensions that are multiples of 8 "
                   "(M=%lld N=%lld K=%lld lda=%lld ldb=%lld ldc=%lld)",
                   (long long)a.M, (long long)a.N, (long long)a.K, (long long)a.lda, (long long)a.ldb, (long long)a.ldc);
  // two-CTA 256 x 256 tiles once there are enough of them to occupy a good part of the SM pairs
  const int64_t pair_tiles = ((a.M + 255) / 256) * ((a.N + 255) / 256);
  if (a.M >= 256 && a.N >= 256 && 4 * pair_tiles >= ctx->sm_count) return launch_bf16_layout<256, true>(ctx, stream, a);
  return launch_bf16_layout<128, false>(ctx, stream, a);
}
