// Tensor-core GEMM for Float32 data on sm_100a: TMA -> shared memory -> tcgen05.mma (TF32, accumulators
// in tensor memory) -> tcgen05.ld epilogue with fused bias / activation / pre-activation store.
//
// fp32 accuracy comes from the error-compensated "3xTF32" scheme.  Operand tiles land in shared memory as raw
// fp32; the tensor core ignores the 13 low mantissa bits of a TF32 operand (measured: clearing them first gives
// bit-identical results), so the raw tile is the "hi" operand and split warps only write lo = x - trunc_tf32(x)
// beside it.  The accumulator receives A_lo*B_hi + A_hi*B_lo + A_hi*B_hi; the dropped lo*lo term is ~2^-20.
//
// Tiles.  One CTA computes a 128 x BN tile of row-major C[M][N] (BN = 256 or 128); or, for large problems, a
// cluster of two CTAs computes a 256 x 256 tile with cta_group::2 MMAs: each CTA loads and splits 128 rows of A
// and 128 columns of B, the leader CTA issues one M = 256 MMA per k-step that reads both CTAs' shared memory,
// and each CTA's tensor memory receives its own 128 rows.  K is walked in blocks of 16 floats through a ring of
// 4-7 stages.  No TMA load is multicast.
//
// The kernel is persistent: one CTA (pair) per SM (pair of SMs) walks the tile grid with stride G, the stage ring
// and the two accumulator buffers run on across tiles, so the epilogue of one tile overlaps the main loop of the
// next and barrier / tensor-memory setup is paid once per launch.
//
// Warp roles: warp 0 issues TMA loads; warp 1 owns tensor memory and issues the MMAs; warps 2-5 are the
// epilogue (one TMEM lane quadrant each); the remaining warps are groups of four split warps (two groups for the
// one-CTA tile, four for the pair) that take k-blocks in turn, so that the latency of one split (load, store,
// proxy fence, arrive) overlaps the splits of the following blocks.
//
// Operands may be K-major (k contiguous) or MN-major (m / n contiguous) in global memory; the shared-memory
// layouts are the canonical ones the MMA descriptors name: 64-byte swizzle for K-major tiles (8 rows x 64 B
// atoms) and, for MN-major tiles, the 128-byte swizzle with 32-byte atoms (128 B x 4 k-rows per atom), which
// is the only MN-major layout the tensor core accepts for 32-bit operands.
//
// The tensor core adds into its fp32 accumulator with truncation, so a long K chain drifts (about 3e-5 of
// max|C| at K = 4096).  K is therefore cut into segments of 2048 that alternate between two accumulator
// buffers in tensor memory: while the MMAs fill one, the epilogue warps drain the other into C with
// round-to-nearest adds.
//
// Every mbarrier wait is bounded; when a wait runs out the kernel records a code in the context's
// device error word, every role leaves its loop, tensor memory is released and the kernel returns.
#include <cuda.h>
#include <stdlib.h>

#include "common.cuh"
#include "tc_common.cuh"

namespace {

constexpr int BM = 128;
constexpr int BK = 16;               // floats per k-block (64 bytes)
constexpr int SEG_KB = 128;          // k-blocks per accumulation segment (2048 k-values)

// Work schedule of one launch.  Tiles [0, dp_tiles) are taken whole: CTA (pair) cid of G takes cid, cid + G, ...
// (n fastest, so the tiles in flight are neighbours and share operand panels in L2).  The remaining tiles - a
// last wave that would leave most SMs idle - are cut along K into units of UNIT_KB k-blocks; the U units are
// dealt out as G contiguous ranges, so a tile may be computed by several CTAs ("parts").  Each part writes its
// partial sums to a workspace slot; the part that finishes last (an atomic ticket per tile, no waiting) adds the
// slots in k order and applies the epilogue.
constexpr int UNIT_KB = 32;
struct Sched {
  int num_tiles, tiles_n, dp_tiles;
  int nu;            // units per tile
  int U;             // units in the tail: (num_tiles - dp_tiles) * nu
  float* ws;         // [2 * G * ranks] slots of BM x 256 floats
  int* tickets;      // [G * ranks * 4], zero between launches
};
struct Portion {
  int tile, kb0, kb1;
  int partial;       // 0: the whole tile, results go to C
  int tail_tile;     // index of the tile inside the tail (partial only)
  int trail;         // 1 when this CTA's range began before the tile's first unit (names the slot)
};
struct WorkIter {
  int w, ta, tb, t0;
  __device__ WorkIter(const Sched& s, int cid, int G) : w(0) {
    ta = t0 = (int)((long long)cid * s.U / G);
    tb = (int)((long long)(cid + 1) * s.U / G);
  }
  __device__ bool next(const Sched& s, int cid, int G, int num_kb, Portion& p) {
    if (w * G + cid < s.dp_tiles) {
      p.tile = w * G + cid; p.kb0 = 0; p.kb1 = num_kb; p.partial = 0; p.tail_tile = 0; p.trail = 0;
      ++w;
      return true;
    }
    if (ta < tb) {
      const int tr = ta / s.nu, ua = ta % s.nu;
      const int rem = tb - ta;
      const int ub = (ua + rem < s.nu) ? ua + rem : s.nu;
      p.tile = s.dp_tiles + tr;
      p.kb0 = ua * UNIT_KB;
      p.kb1 = (ub == s.nu) ? num_kb : ub * UNIT_KB;
      p.partial = (ua == 0 && ub == s.nu) ? 0 : 1;
      p.tail_tile = tr;
      p.trail = (t0 < tr * s.nu) ? 1 : 0;
      ta += ub - ua;
      return true;
    }
    return false;
  }
};

template <int BN, int PASSES, bool PAIR, int SG>
struct Cfg {
  static constexpr int SPLIT_GROUPS = SG;                   // groups of four split warps taking k-blocks in turn
  static_assert(!PAIR || PASSES == 3, "the two-CTA tile exists for the 3-pass scheme only");
  static constexpr int BNC = PAIR ? BN / 2 : BN;            // B columns this CTA loads per stage
  static constexpr int A_BYTES = BM * BK * 4;               // 8 KB
  static constexpr int B_BYTES = BNC * BK * 4;              // 16 KB at 256 columns
  static constexpr int STAGE_BYTES = (PASSES == 3 ? 2 : 1) * (A_BYTES + B_BYTES);
  static constexpr int STAGES = (229376 / STAGE_BYTES) > 8 ? 8 : (229376 / STAGE_BYTES);   // 224 KB of stages at most
  static constexpr int BAR_OFFSET = STAGES * STAGE_BYTES;
  static constexpr int SMEM_BYTES = BAR_OFFSET + 512 + 1024;   // barriers + alignment slack
  static constexpr int TMEM_COLS = 2 * BN;                  // two accumulator buffers
  static constexpr int NUM_WARPS = 6 + (PASSES == 3 ? 4 * SPLIT_GROUPS : 0);
  static constexpr int NUM_THREADS = 32 * NUM_WARPS;
  static constexpr uint32_t ARRIVALS = PAIR ? 8 : 4;        // four warps per CTA arrive on ready / tmem_empty
};

template <bool A_MN, bool B_MN, int BN, int PASSES, bool PAIR, int SG>
__global__ void __launch_bounds__(Cfg<BN, PASSES, PAIR, SG>::NUM_THREADS, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
               float* __restrict__ C, int64_t ldc, float* __restrict__ Z, const float* __restrict__ bias_n, int M,
               int N, int K, int act, int accumulate, int32_t* __restrict__ dev_err, int a3d, int b3d,
               const Sched sch) {
  using cfg = Cfg<BN, PASSES, PAIR, SG>;
  constexpr int SPLIT_GROUPS = SG;
  constexpr int STAGES = cfg::STAGES;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const uint32_t smem_base = smem_u32(smem);
  uint64_t* bars = (uint64_t*)(smem + cfg::BAR_OFFSET);
  const uint32_t bar_base = smem_base + cfg::BAR_OFFSET;
  // barrier slots: full[S], ready[S], empty[S], tmem_full[2], tmem_empty[2]
  auto full_bar = [&](int s) { return bar_base + 8u * (uint32_t)s; };
  auto ready_bar = [&](int s) { return bar_base + 8u * (uint32_t)(STAGES + s); };
  auto empty_bar = [&](int s) { return bar_base + 8u * (uint32_t)(2 * STAGES + s); };
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
  const int tiles_n = sch.tiles_n;
  const int num_kb = (K + BK - 1) / BK;
  // rows of A / C this CTA owns in tile t, the tile's first column, and the first B column this CTA loads
  auto tile_m0 = [&](int t) { return PAIR ? (t / tiles_n) * 256 + 128 * (int)rank : (t / tiles_n) * BM; };
  auto tile_n0 = [&](int t) { return (t % tiles_n) * BN; };

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(ready_bar(s), cfg::ARRIVALS);
      mbar_init(empty_bar(s), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(tmem_full_bar(b), 1);
      mbar_init(tmem_empty_bar(b), cfg::ARRIVALS);
    }
    *s_abort = 0;
    // an error word left set by an earlier launch means: do not start
    s_skip[0] = (*(volatile int32_t*)dev_err != 0) ? 1 : 0;
    s_skip[1] = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    fence_proxy_async();
  }
  if (PAIR) {
    __syncwarp();
    cluster_sync_all();   // both CTAs run and their barriers exist: remote accesses may start
    if (threadIdx.x == 0) {
      // both CTAs of a pair must take the same decision
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
      int m0 = 0, nb0 = 0;
      int it = 0;   // k-blocks issued so far over all tiles: names the stage and its phase
      bool ok = true;
      WorkIter wi(sch, cid, G);
      Portion p;
      while (ok && wi.next(sch, cid, G, num_kb, p)) {
        m0 = tile_m0(p.tile);
        nb0 = tile_n0(p.tile) + (PAIR ? cfg::BNC * (int)rank : 0);
        for (int kb = p.kb0; kb < p.kb1; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (uint32_t)(it / STAGES) & 1u;
          ok = mbar_wait_cluster(empty_bar(s), ph ^ 1u, s_abort);
          if (!ok) break;
          mbar_arrive_expect_tx(full_bar(s), (uint32_t)(cfg::A_BYTES + cfg::B_BYTES));
          const uint32_t a_dst = smem_base + (uint32_t)(s * cfg::STAGE_BYTES);
          const uint32_t b_dst = a_dst + (uint32_t)((PASSES == 3 ? 2 : 1) * cfg::A_BYTES);
          const int k0 = kb * BK;
          if (A_MN) {
            if (a3d) {
              tma_load_3d(a_dst, &tmA, 0, k0, m0 >> 5, full_bar(s));
            } else {
#pragma unroll
              for (int c = 0; c < BM / 32; ++c) tma_load_2d(a_dst + (uint32_t)(c * BK * 128), &tmA, m0 + 32 * c, k0, full_bar(s));
            }
          } else {
            tma_load_2d(a_dst, &tmA, k0, m0, full_bar(s));
          }
          if (B_MN) {
            if (b3d) {
              tma_load_3d(b_dst, &tmB, 0, k0, nb0 >> 5, full_bar(s));
            } else {
#pragma unroll
              for (int c = 0; c < cfg::BNC / 32; ++c) tma_load_2d(b_dst + (uint32_t)(c * BK * 128), &tmB, nb0 + 32 * c, k0, full_bar(s));
            }
          } else {
            tma_load_2d(b_dst, &tmB, k0, nb0, full_bar(s));
          }
        }
      }
    }
  } else if (warp == 1) {
    // -------------------------------------------------- MMA issuer (the leader CTA of a pair) ---
    if (lane == 0 && leader) {
      // instruction descriptor: D = F32, A = B = TF32, operand majors, N >> 3, M >> 4
      const uint32_t idesc = (1u << 4) | (2u << 7) | (2u << 10) | ((A_MN ? 1u : 0u) << 15) | ((B_MN ? 1u : 0u) << 16) |
                             ((uint32_t)(BN >> 3) << 17) | ((uint32_t)((PAIR ? 256 : BM) >> 4) << 24);
      bool ok = true;
      int it = 0, sc = 0;   // k-blocks and accumulation segments issued so far over all tiles
      WorkIter wi(sch, cid, G);
      Portion p;
      while (ok && wi.next(sch, cid, G, num_kb, p))
      for (int kb = p.kb0; kb < p.kb1 && ok; ++kb, ++it) {
        const int s = it % STAGES;
        const uint32_t ph = (uint32_t)(it / STAGES) & 1u;
        const int kb_in_seg = (kb - p.kb0) % SEG_KB;
        const int buf = sc & 1, use = sc >> 1;
        if (kb_in_seg == 0 && use > 0) {
          // the epilogue warps must have drained this accumulator buffer's previous segment
          ok = mbar_wait_cluster(tmem_empty_bar(buf), (uint32_t)(use - 1) & 1u, s_abort);
          if (!ok) break;
        }
        ok = mbar_wait_cluster(PASSES == 3 ? ready_bar(s) : full_bar(s), ph, s_abort);
        if (!ok) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + (uint32_t)(buf * BN);
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
            if (PAIR) {
              tc_mma2_tf32(d_tmem, da_lo, db_hi, idesc, first);
              tc_mma2_tf32(d_tmem, da_hi, db_lo, idesc, 1u);
              tc_mma2_tf32(d_tmem, da_hi, db_hi, idesc, 1u);
            } else {
              tc_mma_tf32(d_tmem, da_lo, db_hi, idesc, first);
              tc_mma_tf32(d_tmem, da_hi, db_lo, idesc, 1u);
              tc_mma_tf32(d_tmem, da_hi, db_hi, idesc, 1u);
            }
          } else {
            tc_mma_tf32(d_tmem, da_hi, db_hi, idesc, first);
          }
        }
        const bool seg_end = (kb_in_seg == SEG_KB - 1 || kb == p.kb1 - 1);
        if (PAIR) {
          tc_commit2_mc(empty_bar(s), (uint16_t)3);                 // frees the stage in both CTAs
          if (seg_end) tc_commit2_mc(tmem_full_bar(buf), (uint16_t)3);
        } else {
          tc_commit(empty_bar(s));
          if (seg_end) tc_commit(tmem_full_bar(buf));
        }
        if (seg_end) ++sc;
      }
    }
  } else if (warp < 6) {
    // -------------------------------------------------------------- epilogue warps ---
    const int q = warp & 3;                 // TMEM lane quadrant this warp may read
    constexpr int RANKS = PAIR ? 2 : 1;
    bool ok = true;
    int sc = 0;                             // segments drained so far over all tiles
    WorkIter wi(sch, cid, G);
    Portion p;
    while (ok && wi.next(sch, cid, G, num_kb, p)) {
      const int n0 = tile_n0(p.tile);
      const int row = tile_m0(p.tile) + 32 * q + lane;
      float* crow = C + (int64_t)row * ldc;
      float* zrow = Z ? Z + (int64_t)row * ldc : nullptr;
      // u: 4 consecutive columns starting at n of this lane's row.  add_c: add what C holds; fin: this is the
      // tile's final value, so bias, pre-activation store and activation apply.
      auto emit4 = [&](float* u, int n, bool add_c, bool fin) {
        if (row >= M) return;
        if (n + 3 < N) {
          if (add_c) {
            const float4 c4 = *(const float4*)(crow + n);
            u[0] += c4.x; u[1] += c4.y; u[2] += c4.z; u[3] += c4.w;
          }
          if (fin) {
            if (bias_n) {
              const float4 b4 = __ldg((const float4*)(bias_n + n));
              u[0] += b4.x; u[1] += b4.y; u[2] += b4.z; u[3] += b4.w;
            }
            if (zrow) *(float4*)(zrow + n) = make_float4(u[0], u[1], u[2], u[3]);
            if (act != FB_ACT_IDENTITY) {
#pragma unroll
              for (int e = 0; e < 4; ++e) u[e] = fb_act_apply(act, u[e]);
            }
          }
          *(float4*)(crow + n) = make_float4(u[0], u[1], u[2], u[3]);
        } else {
          for (int e = 0; e < 4 && n + e < N; ++e) {
            float x = u[e];
            if (add_c) x += crow[n + e];
            if (fin) {
              if (bias_n) x += __ldg(bias_n + n + e);
              if (zrow) zrow[n + e] = x;
              x = fb_act_apply(act, x);
            }
            crow[n + e] = x;
          }
        }
      };
      // A part of a split tile collects its sums in a workspace slot (always 256 floats per row).  The parts of
      // a tile are the CTAs c_first .. c_last whose unit ranges meet it (those with an empty range excepted).
      float* srow = nullptr;
      int c_first = 0, c_last = 0, nparts = 0, rem_first = 0, r_first = 0, u_lo = 0;
      int* ticket = nullptr;
      const int row_off = (32 * q + lane) * 256;
      const int step_q = sch.U / G, step_r = sch.U % G;
      if (p.partial) {
        srow = sch.ws + (size_t)((2 * cid + p.trail) * RANKS + (int)rank) * BM * 256 + row_off;
        u_lo = p.tail_tile * sch.nu;
        const int u_hi = u_lo + sch.nu - 1;
        c_first = (int)(((long long)(u_lo + 1) * G - 1) / sch.U);
        c_last = (int)(((long long)(u_hi + 1) * G - 1) / sch.U);
        ticket = sch.tickets + (c_first * RANKS + (int)rank) * 4 + q;
        // r(pc) = floor(pc * U / G), the first unit of CTA pc, is stepped from c_first on without dividing
        r_first = (int)((long long)c_first * sch.U / G);
        rem_first = (int)((long long)c_first * sch.U % G);
        int r0 = r_first;
        int rem = rem_first;
        for (int pc = c_first; pc <= c_last; ++pc) {
          int r1 = r0 + step_q;
          int rem1 = rem + step_r;
          if (rem1 >= G) { rem1 -= G; ++r1; }
          nparts += (r1 > r0) ? 1 : 0;
          r0 = r1;
          rem = rem1;
        }
      }
      // v[0 .. 4 * NV) += columns [col, col + 4 * NV) of this lane's row summed over parts pc_from .. c_last, in order
      auto add_parts = [&](float* v, int col, int pc_from) {
        int r0 = r_first;
        int rem = rem_first;
        for (int pc = c_first; pc <= c_last; ++pc) {
          int r1 = r0 + step_q;
          int rem1 = rem + step_r;
          if (rem1 >= G) { rem1 -= G; ++r1; }
          if (r1 > r0 && pc >= pc_from) {
            const int tr = (r0 < u_lo) ? 1 : 0;
            const float4* prow =
                (const float4*)(sch.ws + (size_t)((2 * pc + tr) * RANKS + (int)rank) * BM * 256 + row_off + col);
            float4 x[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) x[j] = __ldcg(prow + j);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              v[4 * j] += x[j].x; v[4 * j + 1] += x[j].y; v[4 * j + 2] += x[j].z; v[4 * j + 3] += x[j].w;
            }
          }
          r0 = r1;
          rem = rem1;
        }
      };
      const int nseg = (p.kb1 - p.kb0 + SEG_KB - 1) / SEG_KB;
      bool fused = false;
      for (int seg = 0; seg < nseg && ok; ++seg, ++sc) {
        const int buf = sc & 1, use = sc >> 1;
        ok = mbar_wait_cluster(tmem_full_bar(buf), (uint32_t)use & 1u, s_abort);
        if (!ok) break;
        tc_fence_after();
        // later segments add into what the earlier ones left (round-to-nearest fp32 adds)
        const bool last = (seg == nseg - 1);
        if (p.partial && last && cid == c_first) {
          // The first part of a tile usually finishes last (it is the end of its CTA's range, the other parts are
          // the beginning of theirs).  When every other part has already drawn its ticket, their slots are
          // complete: add them to this last segment on its way out and write C directly.
          int seen = 0;
          if (lane == 0) seen = *(volatile int*)ticket;
          seen = __shfl_sync(0xffffffffu, seen, 0);
          fused = (seen == nparts - 1);
          if (fused) __threadfence();
        }
#pragma unroll 1
        for (int cc = 0; cc < BN / 32; ++cc) {
          const int nb = n0 + cc * 32;
          if (nb >= N) break;   // warp-uniform
          uint32_t r[32];
          tc_ld_32x32b_x32(tmem_base + ((uint32_t)(32 * q) << 16) + (uint32_t)(buf * BN + cc * 32), r);
          tc_wait_ld();
          float* v = reinterpret_cast<float*>(r);
          if (!p.partial) {
            const bool add_c = (seg > 0) || (accumulate != 0);
#pragma unroll
            for (int j = 0; j < 8; ++j) emit4(v + 4 * j, nb + 4 * j, add_c, last);
          } else {
            float4* s4 = (float4*)(srow + cc * 32);
            if (seg > 0) {
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                const float4 o = s4[j];
                v[4 * j] += o.x; v[4 * j + 1] += o.y; v[4 * j + 2] += o.z; v[4 * j + 3] += o.w;
              }
            }
            if (last && fused) {
              add_parts(v, cc * 32, c_first + 1);
              add_parts(v + 16, cc * 32 + 16, c_first + 1);
#pragma unroll
              for (int j = 0; j < 8; ++j) emit4(v + 4 * j, nb + 4 * j, accumulate != 0, true);
            } else {
#pragma unroll
              for (int j = 0; j < 8; ++j) s4[j] = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
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
      if (p.partial && ok) {
        if (fused) {
          __syncwarp();
          if (lane == 0) *ticket = 0;   // every part is accounted for: ready for the next launch
        } else {
          // whoever draws the last ticket adds the slots up, in k order (the same sums as the fused path makes)
          __threadfence();
          __syncwarp();
          int drawn = 0;
          if (lane == 0) drawn = atomicAdd(ticket, 1);
          drawn = __shfl_sync(0xffffffffu, drawn, 0);
          if (drawn == nparts - 1) {
            __threadfence();
#pragma unroll 1
            for (int hc = 0; hc < BN / 16; ++hc) {
              const int nb = n0 + hc * 16;
              if (nb >= N) break;
              float v[16];
#pragma unroll
              for (int j = 0; j < 16; ++j) v[j] = 0.0f;
              add_parts(v, hc * 16, c_first);
#pragma unroll
              for (int j = 0; j < 4; ++j) emit4(v + 4 * j, nb + 4 * j, accumulate != 0, true);
            }
            __syncwarp();
            if (lane == 0) *ticket = 0;   // ready for the next launch
          }
        }
      }
    }
  } else {
    // ------------------------------------------- split warps: write lo = x - trunc_tf32(x) ---
    const int group = (warp - 6) >> 2;
    const int tt = ((warp - 6) & 3) * 32 + lane;   // 0..127 inside the group
    bool ok = true;
    int total_kb = 0;   // the stage ring runs on across tiles
    {
      WorkIter wi(sch, cid, G);
      Portion p;
      while (wi.next(sch, cid, G, num_kb, p)) total_kb += p.kb1 - p.kb0;
    }
    for (int kb = group; kb < total_kb && ok; kb += SPLIT_GROUPS) {
      const int s = kb % STAGES;
      const uint32_t ph = (uint32_t)(kb / STAGES) & 1u;
      ok = mbar_wait(full_bar(s), ph, s_abort);
      if (!ok) break;
      const float4* a_hi = (const float4*)(smem + s * cfg::STAGE_BYTES);
      float4* a_lo = (float4*)(smem + s * cfg::STAGE_BYTES + cfg::A_BYTES);
      const float4* b_hi = (const float4*)(smem + s * cfg::STAGE_BYTES + 2 * cfg::A_BYTES);
      float4* b_lo = (float4*)(smem + s * cfg::STAGE_BYTES + 2 * cfg::A_BYTES + cfg::B_BYTES);
      constexpr int NA = cfg::A_BYTES / 16 / 128, NB = cfg::B_BYTES / 16 / 128;
      float4 v[NA + NB];
#pragma unroll
      for (int i = 0; i < NA; ++i) v[i] = a_hi[tt + i * 128];
#pragma unroll
      for (int i = 0; i < NB; ++i) v[NA + i] = b_hi[tt + i * 128];
#pragma unroll
      for (int i = 0; i < NA + NB; ++i) {
        v[i].x = tf32_lo(v[i].x); v[i].y = tf32_lo(v[i].y); v[i].z = tf32_lo(v[i].z); v[i].w = tf32_lo(v[i].w);
      }
#pragma unroll
      for (int i = 0; i < NA; ++i) a_lo[tt + i * 128] = v[i];
#pragma unroll
      for (int i = 0; i < NB; ++i) b_lo[tt + i * 128] = v[NA + i];
      fence_proxy_async();   // generic-proxy writes become visible to the tensor core's async-proxy reads
      __syncwarp();
      if (lane == 0) {
        if (PAIR) mbar_arrive_cluster(map_to_cta(ready_bar(s), 0u));
        else mbar_arrive(ready_bar(s));
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
  if (threadIdx.x == 0 && *s_abort != 0) atomicExch(dev_err, PAIR ? 1002 : 1001);
}

// --------------------------------------------------------------------------- host side ---
// Workspace of the split-tile schedule, owned by the context: slots for partial sums and the tickets.
struct GemmWorkspace {
  float* ws;
  int* tickets;
};

// 3-d view {32, K, MN / 32} of an MN-major matrix (row k holds MN contiguous floats): box {32, BK, chunks}.
// Only for MN a multiple of 32, so that no chunk straddles the end of a row.
bool encode_map_mn3d(CUtensorMap* map, const float* base, int64_t K, int64_t MN, int64_t ld, uint32_t chunks) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn || MN % 32 != 0) return false;
  cuuint64_t gdim[3] = {32, (cuuint64_t)K, (cuuint64_t)(MN / 32)};
  cuuint64_t gstride[2] = {(cuuint64_t)ld * sizeof(float), 128};
  cuuint32_t box[3] = {32, (cuuint32_t)BK, chunks};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, (void*)base, gdim, gstride, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

template <bool A_MN, bool B_MN, int BN, int PASSES, bool PAIR, int SG>
int32_t launch_variant(fb_ctx* ctx, cudaStream_t stream, const fb_gemm_args& a) {
  using cfg = Cfg<BN, PASSES, PAIR, SG>;
  CUtensorMap tmA, tmB;
  bool ok;
  int a3d = 0, b3d = 0;
  if (A_MN) {
    a3d = encode_map_mn3d(&tmA, a.A, a.K, a.M, a.lda, BM / 32) ? 1 : 0;
    ok = a3d || encode_map(&tmA, a.A, a.K, a.M, a.lda, 32, BK, CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B);
  } else {
    ok = encode_map(&tmA, a.A, a.M, a.K, a.lda, BK, BM, CU_TENSOR_MAP_SWIZZLE_64B);
  }
  if (ok) {
    if (B_MN) {
      b3d = encode_map_mn3d(&tmB, a.B, a.K, a.N, a.ldb, cfg::BNC / 32) ? 1 : 0;
      ok = b3d || encode_map(&tmB, a.B, a.K, a.N, a.ldb, 32, BK, CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B);
    } else {
      ok = encode_map(&tmB, a.B, a.N, a.K, a.ldb, BK, cfg::BNC, CU_TENSOR_MAP_SWIZZLE_64B);
    }
  }
  if (!ok) return fb_fail(FB_ERR_CUDA, "gemm: cuTensorMapEncodeTiled failed (M=%lld N=%lld K=%lld lda=%lld ldb=%lld)",
                          (long long)a.M, (long long)a.N, (long long)a.K, (long long)a.lda, (long long)a.ldb);
  auto kern = gemm_tc_kernel<A_MN, B_MN, BN, PASSES, PAIR, SG>;
  FB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, cfg::SMEM_BYTES));
  // the whole L1 / shared array as shared memory: the communication-stream kernels ask for the same split, and an SM
  // takes CTAs of two kernels together only when their splits agree
  FB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared));
  const int tiles_n = (int)((a.N + BN - 1) / BN);
  const int64_t tiles_m = PAIR ? (a.M + 255) / 256 : (a.M + BM - 1) / BM;
  const int64_t num_tiles = tiles_m * tiles_n;
  if (num_tiles > 0x7fffffff) return fb_fail(FB_ERR_UNSUPPORTED, "gemm: too many tiles");
  // one CTA (pair) per SM (pair of SMs)
  // (fewer when the caller reserved SMs for communication kernels that run beside this one: a persistent grid that
  // does not fit waits for them to finish)
  const int sms = ctx->sm_count - ctx->reserved_sms;
  const int64_t Gmax = PAIR ? (sms / 2 > 0 ? sms / 2 : 1) : sms;
  const int num_kb = (int)((a.K + BK - 1) / BK);
  Sched sch;
  sch.num_tiles = (int)num_tiles;
  sch.tiles_n = tiles_n;
  sch.dp_tiles = (int)num_tiles;
  sch.nu = (num_kb + UNIT_KB - 1) / UNIT_KB;
  sch.U = 0;
  sch.ws = nullptr;
  sch.tickets = nullptr;
  int64_t G = Gmax < num_tiles ? Gmax : num_tiles;
  // A last wave that fills less than 3/4 of the machine is cut along K and spread over all CTAs.  (Fuller waves
  // gain nothing: the kernel runs at the power limit, where idle SMs let the busy ones clock higher.)
  const int64_t rest = num_tiles % Gmax;
  const GemmWorkspace* gw = (const GemmWorkspace*)ctx->gemm_ws;
  if (rest != 0 && 4 * rest < 3 * Gmax && sch.nu > 1 && rest * sch.nu < 0x40000000 && gw != nullptr) {
    sch.dp_tiles = (int)(num_tiles - rest);
    sch.U = (int)(rest * sch.nu);
    sch.ws = gw->ws;
    sch.tickets = gw->tickets;
    G = Gmax;
  }
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
  FB_CUDA(cudaLaunchKernelEx(&lc, kern, tmA, tmB, a.C, a.ldc, a.Z, a.bias_n, (int)a.M, (int)a.N, (int)a.K, a.act,
                             a.accumulate, ctx->dev_error, a3d, b3d, sch));
  FB_LAUNCH_CHECK();
  return FB_OK;
}

template <int BN, int PASSES, bool PAIR, int SG>
int32_t launch_layout_sg(fb_ctx* ctx, cudaStream_t stream, const fb_gemm_args& a) {
  if (a.a_mn_major) {
    if (a.b_mn_major) return launch_variant<true, true, BN, PASSES, PAIR, SG>(ctx, stream, a);
    return launch_variant<true, false, BN, PASSES, PAIR, SG>(ctx, stream, a);
  }
  if (a.b_mn_major) return launch_variant<false, true, BN, PASSES, PAIR, SG>(ctx, stream, a);
  return launch_variant<false, false, BN, PASSES, PAIR, SG>(ctx, stream, a);
}

// Split-warp groups: the one-CTA tile is bound by shared-memory bandwidth and gains nothing beyond two groups; the
// two-CTA tile is bound by the latency of one split (wait, load, store, proxy fence, remote arrive) and keeps
// gaining up to four (measured 157 -> 175 -> 182 TFLOP/s for 2 -> 3 -> 4 groups at 4096^3).
template <int BN, int PASSES, bool PAIR>
int32_t launch_layout(fb_ctx* ctx, cudaStream_t stream, const fb_gemm_args& a) {
  return launch_layout_sg<BN, PASSES, PAIR, (PAIR ? 4 : 2)>(ctx, stream, a);
}

// Measured on B200 (4096^3, 3xTF32, persistent kernels): one-CTA 128 x 256 tiles 200-213 TFLOP/s (every MMA re-reads
// all 256 B columns from shared memory), two-CTA 256 x 256 tiles 215-232 TFLOP/s (each CTA reads only its 128 B
// columns).  At 1024 x 4096 x 4096 (one wave of 64 two-CTA tiles on 74 SM pairs) both, and cutting every tile along
// K over all pairs, take 0.204-0.207 ms: what is left there is the unoverlapped prologue and epilogue of a single tile.
}  // namespace

bool fb_gemm_tc_supported(const fb_gemm_args& a) {
  if (a.M < 1 || a.N < 1 || a.K < 1) return false;
  if (a.M > 0x7fffff00 || a.N > 0x7fffff00 || a.K > 0x7fffff00) return false;
  if (a.bias_m != nullptr) return false;
  if (!fb_aligned16(a.A) || !fb_aligned16(a.B) || !fb_aligned16(a.C)) return false;
  if (a.Z && !fb_aligned16(a.Z)) return false;
  if (a.bias_n && !fb_aligned16(a.bias_n)) return false;
  if (a.lda % 4 || a.ldb % 4 || a.ldc % 4) return false;
  // the leading dimension must cover the contiguous extent
  if (a.lda < (a.a_mn_major ? a.M : a.K) || a.ldb < (a.b_mn_major ? a.N : a.K) || a.ldc < a.N) return false;
  return true;
}

// passes: 3 = 3xTF32, 1 = one TF32 pass, 32 = 3xTF32 on two-CTA tiles where the shape allows
int32_t fb_gemm_tc_launch(fb_ctx* ctx, cudaStream_t stream, const fb_gemm_args& a, int passes) {
  if (!fb_gemm_tc_supported(a)) return FB_ERR_UNSUPPORTED;
  const bool passes_flag_pair = (passes == 32);
  if (passes_flag_pair) passes = 3;
  // 128 x 256 tiles unless they would leave most of the machine idle: the wider tile does twice the MMA work per
  // split / barrier round trip, so one 86 %-full wave of them beats two waves of 128 x 128 tiles
  const int64_t tiles256 = ((a.M + BM - 1) / BM) * ((a.N + 255) / 256);
  const bool narrow = (a.N <= 128) || (2 * tiles256 <= ctx->sm_count);
  if (passes == 3) {
    // two-CTA 256 x 256 tiles once there are enough of them to occupy a good part of the SM pairs
    const int64_t pair_tiles = ((a.M + 255) / 256) * ((a.N + 255) / 256);
    if (a.M >= 256 && a.N >= 256 && (passes_flag_pair || 4 * pair_tiles >= ctx->sm_count))
      return launch_layout<256, 3, true>(ctx, stream, a);
    if (narrow) return launch_layout<128, 3, false>(ctx, stream, a);
    return launch_layout<256, 3, false>(ctx, stream, a);
  }
  if (narrow) return launch_layout<128, 1, false>(ctx, stream, a);
  return launch_layout<256, 1, false>(ctx, stream, a);
}

// Called by fb_ctx_create / fb_ctx_destroy.  The workspace is allocated up front (2 slots of 128 x 256 floats per
// SM, 37 MiB on 148 SMs) so that no launch allocates; calls that share a context must be ordered on one stream.
int32_t fb_gemm_workspace_create(fb_ctx* ctx) {
  GemmWorkspace* gw = new GemmWorkspace();
  gw->ws = nullptr;
  gw->tickets = nullptr;
  const size_t slots = (size_t)2 * (size_t)ctx->sm_count;
  const size_t tickets = (size_t)ctx->sm_count * 4;
  if (cudaMalloc(&gw->ws, slots * BM * 256 * sizeof(float)) != cudaSuccess ||
      cudaMalloc(&gw->tickets, tickets * sizeof(int)) != cudaSuccess) {
    cudaGetLastError();
    if (gw->ws) cudaFree(gw->ws);
    delete gw;
    return fb_fail(FB_ERR_ALLOC, "fb_ctx_create: GEMM workspace allocation failed");
  }
  cudaMemset(gw->tickets, 0, tickets * sizeof(int));
  ctx->gemm_ws = gw;
  return FB_OK;
}

void fb_gemm_workspace_reset(fb_ctx* ctx, cudaStream_t stream) {
  GemmWorkspace* gw = (GemmWorkspace*)ctx->gemm_ws;
  if (gw != nullptr && gw->tickets != nullptr) cudaMemsetAsync(gw->tickets, 0, (size_t)ctx->sm_count * 4 * sizeof(int), stream);
}

void fb_gemm_workspace_destroy(fb_ctx* ctx) {
  GemmWorkspace* gw = (GemmWorkspace*)ctx->gemm_ws;
  if (gw == nullptr) return;
  if (gw->ws) cudaFree(gw->ws);
  if (gw->tickets) cudaFree(gw->tickets);
  delete gw;
  ctx->gemm_ws = nullptr;
}
