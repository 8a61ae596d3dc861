// Flash-style attention forward on the tensor cores for Float32 data (head size 64): S = Q K' and O += P V are
// tcgen05 TF32 MMAs with the error-compensated 3-pass split (hi / lo operands), the online softmax runs on the
// accumulator read back from tensor memory, and no L x L array ever exists in HBM.
//
// One CTA owns 128 queries of one (batch, head) and walks the keys in blocks of 64:
//   warp 0      TMA producer: the Q tile once, then a K and a V tile per block (single-buffered; a tile is reloaded
//               as soon as the MMAs that read it have completed)
//   warp 1      owns tensor memory (128 columns: S in 0..63, P V in 64..127) and issues the MMAs
//   warps 2-5   softmax: thread = one query row (its TMEM lane).  Reads S, keeps the running maximum and sum,
//               writes P (raw value = hi operand, and lo = p - tf32(p)) to shared memory in the K-major 64-byte
//               swizzled layout the MMA descriptor names, then adds P V (read back from tensor memory) to its
//               64 output accumulators with round-to-nearest adds
//   warps 6-9   split warps: write the lo = x - tf32(x) twin of every Q / K / V tile beside the raw tile
//
// Shared-memory tiles use the layouts already proven by the GEMM: K-major chunks of 16 floats with the 64-byte
// swizzle for Q, K and P; the 128-byte swizzle with 32-byte atoms for the MN-major V tile (keys are its K rows).
// Every mbarrier wait is bounded; when one runs out the kernel records 4001 in the context's device error word,
// all roles leave their loops, tensor memory is released and the kernel returns.
#include <cuda.h>
#include <stdlib.h>

#include "common.cuh"
#include "tc_common.cuh"

namespace {

constexpr int QT = 128;   // queries per CTA
constexpr int KT = 64;    // keys per block
constexpr int HD = 64;    // head size (q/k features and v features per head)
constexpr int ATC_THREADS = 320;

__device__ __forceinline__ void tc_st_32x32b_x32(uint32_t taddr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
      "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]),
      "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]),
      "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tc_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// D[tmem] (+)= A[tmem] * B[smem]: the A tile (128 rows x 8 TF32 values) sits in 8 consecutive TMEM columns
__device__ __forceinline__ void tc_mma_tf32_ta(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], [%1], %2, %3, {%5, %6, %7, %8}, p;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(0u), "r"(0u), "r"(0u), "r"(0u)
      : "memory");
}

// 2^x by the special-function unit (relative error ~2^-22, far inside the tolerance of a softmax weight)
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

struct AtcDims {
  int64_t E, Ev, Lq, Lk;
  int H, causal;
  float scale_log2;   // log2(e) / sqrt(d)
  float scale;        // 1 / sqrt(d)
};

// Pipelined variant: three K / V stages in shared memory (a K tile is reloaded three blocks ahead, which covers the
// latency of its TMA load); Q lives in tensor memory as the A operand of Q K' (hi and lo parts, stored once by the
// softmax warps), next to two S buffers (P hi overwrites S in place), two P lo buffers and two P V buffers.  The MMA
// warp issues Q K' of block j + 1 before P V of block j, so the tensor pipe works on the next scores while the softmax
// warps are busy with the current ones; the softmax warps add P V of block j - 1 after they have handed P of block j
// to the tensor core.
//   TMEM columns: Q hi 0..63, Q lo 64..127; S/P_hi 128.., 192..; P_lo 256.., 320..; P V 384.., 448..
constexpr int P2_NSTAGE = 3;
constexpr int P2_STAGE0 = 0, P2_STAGE_BYTES = 65536;          // per stage: K hi, K lo, V hi, V lo (16 KB each)
constexpr int P2_BAR = P2_STAGE0 + P2_NSTAGE * P2_STAGE_BYTES;   // 196608
constexpr int ATC2_SMEM = P2_BAR + 512 + 1024;
enum { C_QREADY = 0, C_KFULL, C_KREADY = C_KFULL + 3, C_KFREE = C_KREADY + 3, C_VFULL = C_KFREE + 3, C_VREADY = C_VFULL + 3,
       C_VFREE = C_VREADY + 3, C_SFULL = C_VFREE + 3, C_PREADY = C_SFULL + 2, C_OFULL = C_PREADY + 2, C_COUNT = C_OFULL + 2 };

__global__ void __launch_bounds__(ATC_THREADS, 1)
attn_fwd_tc2_kernel(const float* __restrict__ qmat, const __grid_constant__ CUtensorMap tmK,
                    const __grid_constant__ CUtensorMap tmV, float* __restrict__ o, float* __restrict__ lse, AtcDims D,
                    int32_t* __restrict__ dev_err) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const uint32_t sb = smem_u32(smem);
  const uint32_t bar0 = sb + P2_BAR;
  auto bar = [&](int i) { return bar0 + 8u * (uint32_t)i; };
  volatile uint32_t* s_tmem = (volatile uint32_t*)(smem + P2_BAR + 8 * C_COUNT);
  volatile int* s_abort = (volatile int*)(smem + P2_BAR + 8 * C_COUNT + 8);
  volatile int* s_skip = (volatile int*)(smem + P2_BAR + 8 * C_COUNT + 16);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // causal: the last query tiles have the most key blocks, so they are scheduled first
  const int64_t i0 = (int64_t)(D.causal ? gridDim.x - 1 - blockIdx.x : blockIdx.x) * QT;
  const int h = blockIdx.y;
  const int64_t b = blockIdx.z;
  int64_t kv_end = D.Lk;
  if (D.causal && i0 + QT < kv_end) kv_end = i0 + QT;
  const int nkb = (int)((kv_end + KT - 1) / KT);

  if (threadIdx.x == 0) {
    mbar_init(bar(C_QREADY), 4);
    for (int st = 0; st < P2_NSTAGE; ++st) {
      mbar_init(bar(C_KFULL + st), 1);
      mbar_init(bar(C_KREADY + st), 4);
      mbar_init(bar(C_KFREE + st), 1);
      mbar_init(bar(C_VFULL + st), 1);
      mbar_init(bar(C_VREADY + st), 4);
      mbar_init(bar(C_VFREE + st), 1);
    }
    for (int st = 0; st < 2; ++st) {
      mbar_init(bar(C_SFULL + st), 1);
      mbar_init(bar(C_PREADY + st), 4);
      mbar_init(bar(C_OFULL + st), 1);
    }
    *s_abort = 0;
    *s_skip = (*(volatile int32_t*)dev_err != 0) ? 1 : 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    fence_proxy_async();
  }
  __syncthreads();
  if (*s_skip != 0) return;
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32((const void*)s_tmem)), "r"(512u)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *s_tmem;
  // block j uses TMEM buffer j & 1 for the (j >> 1)-th time and shared-memory stage j % 3 for the (j / 3)-th time
  auto par = [](int j) { return (uint32_t)(j >> 1) & 1u; };
  auto par3 = [](int j) { return (uint32_t)(j / P2_NSTAGE) & 1u; };

  if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer ---
    if (lane == 0) {
      const int krow0 = (int)(b * D.Lk);
      for (int j = 0; j < nkb; ++j) {
        const int st = j % P2_NSTAGE;
        const uint32_t base = sb + P2_STAGE0 + (uint32_t)(st * P2_STAGE_BYTES);
        if (j >= P2_NSTAGE && !mbar_wait(bar(C_KFREE + st), par3(j - P2_NSTAGE), s_abort)) break;
        mbar_arrive_expect_tx(bar(C_KFULL + st), 16384u);
#pragma unroll
        for (int c = 0; c < 4; ++c) tma_load_2d(base + c * 4096, &tmK, h * HD + 16 * c, krow0 + j * KT, bar(C_KFULL + st));
        if (j >= P2_NSTAGE && !mbar_wait(bar(C_VFREE + st), par3(j - P2_NSTAGE), s_abort)) break;
        mbar_arrive_expect_tx(bar(C_VFULL + st), 16384u);
        tma_load_3d(base + 32768, &tmV, 0, krow0 + j * KT, 2 * h, bar(C_VFULL + st));
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer ---
    if (lane == 0) {
      const uint32_t idesc_qk = (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(KT >> 3) << 17) | ((uint32_t)(QT >> 4) << 24);
      const uint32_t idesc_pv = idesc_qk | (1u << 16);
      // descriptors differ only in their 14-bit start-address field (units of 16 bytes): build one per tile and add
      // the per-k-step offsets, so that issuing an MMA costs a couple of integer adds
      auto issue_qk = [&](int j) -> bool {
        const int st = j % P2_NSTAGE, buf = j & 1;
        if (!mbar_wait(bar(C_KREADY + st), par3(j), s_abort)) return false;
        tc_fence_after();
        const uint32_t kb = sb + P2_STAGE0 + (uint32_t)(st * P2_STAGE_BYTES);
        const uint64_t dk_hi = make_smem_desc(kb, 16, 512, LAYOUT_SW64), dk_lo = make_smem_desc(kb + 16384, 16, 512, LAYOUT_SW64);
        const uint32_t d = tmem_base + 128u + (uint32_t)(64 * buf);
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
          const uint64_t ko = (uint64_t)(((ks >> 1) * 4096 + (ks & 1) * 32) >> 4);
          const uint32_t ao = (uint32_t)(8 * ks);
          tc_mma_tf32_ta(d, tmem_base + 64u + ao, dk_hi + ko, idesc_qk, ks > 0 ? 1u : 0u);
          tc_mma_tf32_ta(d, tmem_base + ao, dk_lo + ko, idesc_qk, 1u);
          tc_mma_tf32_ta(d, tmem_base + ao, dk_hi + ko, idesc_qk, 1u);
        }
        tc_commit(bar(C_SFULL + buf));
        tc_commit(bar(C_KFREE + st));
        return true;
      };
      bool ok = mbar_wait(bar(C_QREADY), 0u, s_abort);
      ok = ok && issue_qk(0);
      for (int j = 0; j < nkb && ok; ++j) {
        const int st = j % P2_NSTAGE, buf = j & 1;
        if (j + 1 < nkb) {
          ok = issue_qk(j + 1);
          if (!ok) break;
        }
        ok = mbar_wait(bar(C_PREADY + buf), par(j), s_abort) && mbar_wait(bar(C_VREADY + st), par3(j), s_abort);
        if (!ok) break;
        tc_fence_after();
        const uint32_t vb = sb + P2_STAGE0 + (uint32_t)(st * P2_STAGE_BYTES) + 32768;
        const uint32_t d = tmem_base + 384u + (uint32_t)(64 * buf);
        const uint64_t dv_hi = make_smem_desc(vb, KT * 128, 512, LAYOUT_SW128_32B);
        const uint64_t dv_lo = make_smem_desc(vb + 16384, KT * 128, 512, LAYOUT_SW128_32B);
        const uint32_t a_hi0 = tmem_base + 128u + (uint32_t)(64 * buf), a_lo0 = a_hi0 + 128u;
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
          const uint64_t vo = (uint64_t)((ks * 1024) >> 4);
          tc_mma_tf32_ta(d, a_lo0 + (uint32_t)(8 * ks), dv_hi + vo, idesc_pv, ks > 0 ? 1u : 0u);
          tc_mma_tf32_ta(d, a_hi0 + (uint32_t)(8 * ks), dv_lo + vo, idesc_pv, 1u);
          tc_mma_tf32_ta(d, a_hi0 + (uint32_t)(8 * ks), dv_hi + vo, idesc_pv, 1u);
        }
        tc_commit(bar(C_OFULL + buf));
        tc_commit(bar(C_VFREE + st));
      }
    }
  } else if (warp < 6) {
    // ------------------------------------------------------------------ softmax warps ---
    const int q = warp & 3;
    const int row = 32 * q + lane;
    const int64_t gi = i0 + row;
    const uint32_t t_row = tmem_base + ((uint32_t)(32 * q) << 16);
    float m = -INFINITY, l = 0.0f;
    float acc[HD];
#pragma unroll
    for (int c = 0; c < HD; ++c) acc[c] = 0.0f;
    bool ok = true;
    {
      // Q row of this thread into tensor memory: the raw value is the hi operand, lo = x - tf32(x)
      const float* src = qmat + (b * D.Lq + gi) * D.E + (int64_t)h * HD;
#pragma unroll
      for (int hf = 0; hf < 2; ++hf) {
        uint32_t hi[32], lo[32];
#pragma unroll
        for (int c4 = 0; c4 < 8; ++c4) {
          float4 x = make_float4(0.f, 0.f, 0.f, 0.f);
          if (gi < D.Lq) x = __ldg((const float4*)(src + 32 * hf + 4 * c4));
          hi[4 * c4] = __float_as_uint(x.x); hi[4 * c4 + 1] = __float_as_uint(x.y);
          hi[4 * c4 + 2] = __float_as_uint(x.z); hi[4 * c4 + 3] = __float_as_uint(x.w);
          lo[4 * c4] = __float_as_uint(tf32_lo(x.x)); lo[4 * c4 + 1] = __float_as_uint(tf32_lo(x.y));
          lo[4 * c4 + 2] = __float_as_uint(tf32_lo(x.z)); lo[4 * c4 + 3] = __float_as_uint(tf32_lo(x.w));
        }
        tc_st_32x32b_x32(t_row + (uint32_t)(32 * hf), hi);
        tc_st_32x32b_x32(t_row + (uint32_t)(64 + 32 * hf), lo);
      }
      tc_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(C_QREADY));
    }
    // adds P V of block jj to the accumulators (waits for its MMAs)
    auto add_pv = [&](int jj) -> bool {
      const int st = jj & 1;
      if (!mbar_wait(bar(C_OFULL + st), par(jj), s_abort)) return false;
      tc_fence_after();
      uint32_t v0[32], v1[32];
      tc_ld_32x32b_x32(t_row + 384u + (uint32_t)(64 * st), v0);
      tc_ld_32x32b_x32(t_row + 416u + (uint32_t)(64 * st), v1);
      tc_wait_ld();
#pragma unroll
      for (int c = 0; c < 32; ++c) {
        acc[c] += __uint_as_float(v0[c]);
        acc[c + 32] += __uint_as_float(v1[c]);
      }
      return true;
    };
    for (int j = 0; j < nkb && ok; ++j) {
      const int st = j & 1;
      const int64_t j0 = (int64_t)j * KT;
      ok = mbar_wait(bar(C_SFULL + st), par(j), s_abort);
      if (!ok) break;
      tc_fence_after();
      uint32_t s0[32], s1[32];
      const uint32_t t_s = t_row + 128u + (uint32_t)(64 * st);
      tc_ld_32x32b_x32(t_s, s0);
      tc_ld_32x32b_x32(t_s + 32u, s1);
      tc_wait_ld();
      int64_t lim = D.Lk - j0;
      if (D.causal && gi - j0 + 1 < lim) lim = gi - j0 + 1;
      const int nvalid = lim < 0 ? 0 : (lim > KT ? KT : (int)lim);
      // keys the query may not see get a score of -inf (whole blocks below the diagonal need no test)
      if (nvalid < KT) {
#pragma unroll
        for (int c = 0; c < 32; ++c) {
          if (c >= nvalid) s0[c] = 0xff800000u;
          if (c + 32 >= nvalid) s1[c] = 0xff800000u;
        }
      }
      float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
      for (int c = 0; c < 32; ++c) {
        mx0 = fmaxf(mx0, __uint_as_float(s0[c]));
        mx1 = fmaxf(mx1, __uint_as_float(s1[c]));
      }
      const float m_new = fmaxf(m, fmaxf(mx0, mx1));
      const float m_use = (m_new == -INFINITY) ? 0.0f : m_new;
      const float alpha = fast_exp2((m - m_use) * D.scale_log2);   // m = -inf gives 0
      const float mc = m_use * D.scale_log2;
      float rs0 = 0.0f, rs1 = 0.0f;
      {
        // P = 2^(s c - m c) over S in place (the raw value is the hi operand) and its lo part, 32 columns at a time
        uint32_t lo[32];
#pragma unroll
        for (int c = 0; c < 32; ++c) {
          const float p0 = fast_exp2(fmaf(__uint_as_float(s0[c]), D.scale_log2, -mc));
          rs0 += p0;
          s0[c] = __float_as_uint(p0);
          lo[c] = __float_as_uint(tf32_lo(p0));
        }
        tc_st_32x32b_x32(t_s, s0);
        tc_st_32x32b_x32(t_s + 128u, lo);
#pragma unroll
        for (int c = 0; c < 32; ++c) {
          const float p1 = fast_exp2(fmaf(__uint_as_float(s1[c]), D.scale_log2, -mc));
          rs1 += p1;
          s1[c] = __float_as_uint(p1);
          lo[c] = __float_as_uint(tf32_lo(p1));
        }
        tc_st_32x32b_x32(t_s + 32u, s1);
        tc_st_32x32b_x32(t_s + 160u, lo);
        tc_wait_st();
      }
      const float rs = rs0 + rs1;
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(C_PREADY + st));
      // the previous block's P V joins the accumulators before they are rescaled for this block
      if (j > 0) {
        ok = add_pv(j - 1);
        if (!ok) break;
      }
      l = l * alpha + rs;
      m = m_new;
      if (alpha != 1.0f) {   // the running maximum moved (rare after the first blocks)
#pragma unroll
        for (int c = 0; c < HD; ++c) acc[c] *= alpha;
      }
    }
    if (ok) ok = add_pv(nkb - 1);
    if (ok && gi < D.Lq) {
      const float inv = l > 0.0f ? 1.0f / l : 0.0f;
      float* orow = o + (b * D.Lq + gi) * D.Ev + (int64_t)h * HD;
#pragma unroll
      for (int c = 0; c < HD; c += 4)
        *(float4*)(orow + c) = make_float4(acc[c] * inv, acc[c + 1] * inv, acc[c + 2] * inv, acc[c + 3] * inv);
      lse[(b * D.H + h) * D.Lq + gi] = (l > 0.0f) ? m * D.scale + logf(l) : -INFINITY;
    }
  } else {
    // --------------------------------------------- split warps: lo = x - tf32(x) twins ---
    const int tt = (warp - 6) * 32 + lane;
    auto split = [&](int off_hi, int off_lo, int n16) {
      const float4* hi = (const float4*)(smem + off_hi);
      float4* lo = (float4*)(smem + off_lo);
      for (int i = 0; i < n16; ++i) {
        float4 v = hi[tt + i * 128];
        v.x = tf32_lo(v.x); v.y = tf32_lo(v.y); v.z = tf32_lo(v.z); v.w = tf32_lo(v.w);
        lo[tt + i * 128] = v;
      }
      fence_proxy_async();
      __syncwarp();
    };
    bool ok = true;
    for (int j = 0; j < nkb && ok; ++j) {
      const int st = j % P2_NSTAGE;
      const int base = P2_STAGE0 + st * P2_STAGE_BYTES;
      ok = mbar_wait(bar(C_KFULL + st), par3(j), s_abort);
      if (!ok) break;
      split(base, base + 16384, 8);
      if (lane == 0) mbar_arrive(bar(C_KREADY + st));
      ok = mbar_wait(bar(C_VFULL + st), par3(j), s_abort);
      if (!ok) break;
      split(base + 32768, base + 49152, 8);
      if (lane == 0) mbar_arrive(bar(C_VREADY + st));
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
  }
  if (threadIdx.x == 0 && *s_abort != 0) atomicExch(dev_err, 4002);
}

// ------------------------------------------------------------------------------------------------------------------
// dQ of the attention backward pass on the tensor cores.  One CTA owns 128 queries of one (batch, head); Q and dO of
// those queries live in tensor memory for the whole kernel (hi and lo parts, A operands of the MMAs).  For every
// block of 64 keys: S = Q K' and dP = dO V' (B operands: K and V tiles, K-major), the compute warps turn them into
// dS = P (dP - delta) with P = exp(S / sqrt(d) - lse) and hand dS back through tensor memory, and dQ += dS K (B
// operand: the same K tile loaded a second time in the MN-major layout, keys being its K rows).  dQ accumulates in
// tensor memory over at most 32 blocks (2048 keys, the accumulation length the GEMM also uses).
//   TMEM columns: Q hi 0, Q lo 64, dO hi 128, dO lo 192, S -> dS hi 256, dS lo 320, dP 384, dQ 448
constexpr int DQ_STAGE_BYTES = 98304;   // K k-major hi/lo (32 KB), K mn-major hi/lo (32 KB), V k-major hi/lo (32 KB)
constexpr int DQ_BAR = 2 * DQ_STAGE_BYTES;
constexpr int DQ_SMEM = DQ_BAR + 256 + 1024;
constexpr int DQ_MAX_BLOCKS = 32;
enum { E_QREADY = 0, E_FULL, E_READY = E_FULL + 2, E_FREE = E_READY + 2, E_SFULL = E_FREE + 2, E_DSREADY, E_DQFULL, E_COUNT };

__global__ void __launch_bounds__(ATC_THREADS, 1)
attn_bwd_dq_tc_kernel(const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmKmn,
                      const __grid_constant__ CUtensorMap tmV, const float* __restrict__ q, const float* __restrict__ dout,
                      const float* __restrict__ lse, const float* __restrict__ dlt, float* __restrict__ dq, AtcDims D,
                      int32_t* __restrict__ dev_err) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const uint32_t sb = smem_u32(smem);
  const uint32_t bar0 = sb + DQ_BAR;
  auto bar = [&](int i) { return bar0 + 8u * (uint32_t)i; };
  volatile uint32_t* s_tmem = (volatile uint32_t*)(smem + DQ_BAR + 8 * E_COUNT);
  volatile int* s_abort = (volatile int*)(smem + DQ_BAR + 8 * E_COUNT + 8);
  volatile int* s_skip = (volatile int*)(smem + DQ_BAR + 8 * E_COUNT + 16);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t i0 = (int64_t)(D.causal ? gridDim.x - 1 - blockIdx.x : blockIdx.x) * QT;
  const int h = blockIdx.y;
  const int64_t b = blockIdx.z;
  int64_t kv_end = D.Lk;
  if (D.causal && i0 + QT < kv_end) kv_end = i0 + QT;
  const int nkb = (int)((kv_end + KT - 1) / KT);

  if (threadIdx.x == 0) {
    mbar_init(bar(E_QREADY), 4);
    for (int st = 0; st < 2; ++st) {
      mbar_init(bar(E_FULL + st), 1);
      mbar_init(bar(E_READY + st), 4);
      mbar_init(bar(E_FREE + st), 1);
    }
    mbar_init(bar(E_SFULL), 1);
    mbar_init(bar(E_DSREADY), 4);
    mbar_init(bar(E_DQFULL), 1);
    *s_abort = 0;
    *s_skip = (*(volatile int32_t*)dev_err != 0) ? 1 : 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    fence_proxy_async();
  }
  __syncthreads();
  if (*s_skip != 0) return;
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32((const void*)s_tmem)), "r"(512u)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *s_tmem;
  auto par = [](int j) { return (uint32_t)(j >> 1) & 1u; };

  if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer ---
    if (lane == 0) {
      const int krow0 = (int)(b * D.Lk);
      for (int j = 0; j < nkb; ++j) {
        const int st = j & 1;
        const uint32_t base = sb + (uint32_t)(st * DQ_STAGE_BYTES);
        if (j >= 2 && !mbar_wait(bar(E_FREE + st), par(j - 2), s_abort)) break;
        mbar_arrive_expect_tx(bar(E_FULL + st), 49152u);
#pragma unroll
        for (int c = 0; c < 4; ++c) tma_load_2d(base + c * 4096, &tmK, h * HD + 16 * c, krow0 + j * KT, bar(E_FULL + st));
        tma_load_3d(base + 32768, &tmKmn, 0, krow0 + j * KT, 2 * h, bar(E_FULL + st));
#pragma unroll
        for (int c = 0; c < 4; ++c) tma_load_2d(base + 65536 + c * 4096, &tmV, h * HD + 16 * c, krow0 + j * KT, bar(E_FULL + st));
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer ---
    if (lane == 0) {
      const uint32_t idesc_kk = (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(KT >> 3) << 17) | ((uint32_t)(QT >> 4) << 24);
      const uint32_t idesc_mn = idesc_kk | (1u << 16);   // N = 64 either way (keys, or features of dQ)
      const uint32_t t_q = tmem_base, t_do = tmem_base + 128u, t_s = tmem_base + 256u, t_dp = tmem_base + 384u, t_dq = tmem_base + 448u;
      bool ok = mbar_wait(bar(E_QREADY), 0u, s_abort);
      for (int j = 0; j < nkb && ok; ++j) {
        const int st = j & 1;
        ok = mbar_wait(bar(E_READY + st), par(j), s_abort);
        if (!ok) break;
        tc_fence_after();
        const uint32_t base = sb + (uint32_t)(st * DQ_STAGE_BYTES);
        const uint64_t dk_hi = make_smem_desc(base, 16, 512, LAYOUT_SW64), dk_lo = make_smem_desc(base + 16384, 16, 512, LAYOUT_SW64);
        const uint64_t dv_hi = make_smem_desc(base + 65536, 16, 512, LAYOUT_SW64), dv_lo = make_smem_desc(base + 81920, 16, 512, LAYOUT_SW64);
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {   // S = Q K' and dP = dO V' over the 64 features
          const uint64_t bo = (uint64_t)(((ks >> 1) * 4096 + (ks & 1) * 32) >> 4);
          const uint32_t ao = (uint32_t)(8 * ks);
          tc_mma_tf32_ta(t_s, t_q + 64u + ao, dk_hi + bo, idesc_kk, ks > 0 ? 1u : 0u);
          tc_mma_tf32_ta(t_s, t_q + ao, dk_lo + bo, idesc_kk, 1u);
          tc_mma_tf32_ta(t_s, t_q + ao, dk_hi + bo, idesc_kk, 1u);
          tc_mma_tf32_ta(t_dp, t_do + 64u + ao, dv_hi + bo, idesc_kk, ks > 0 ? 1u : 0u);
          tc_mma_tf32_ta(t_dp, t_do + ao, dv_lo + bo, idesc_kk, 1u);
          tc_mma_tf32_ta(t_dp, t_do + ao, dv_hi + bo, idesc_kk, 1u);
        }
        tc_commit(bar(E_SFULL));
        ok = mbar_wait(bar(E_DSREADY), (uint32_t)j & 1u, s_abort);
        if (!ok) break;
        tc_fence_after();
        const uint64_t dm_hi = make_smem_desc(base + 32768, KT * 128, 512, LAYOUT_SW128_32B);
        const uint64_t dm_lo = make_smem_desc(base + 49152, KT * 128, 512, LAYOUT_SW128_32B);
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {   // dQ += dS K over the 64 keys
          const uint64_t bo = (uint64_t)((ks * 1024) >> 4);
          const uint32_t ao = (uint32_t)(8 * ks);
          tc_mma_tf32_ta(t_dq, t_s + 64u + ao, dm_hi + bo, idesc_mn, (j > 0 || ks > 0) ? 1u : 0u);
          tc_mma_tf32_ta(t_dq, t_s + ao, dm_lo + bo, idesc_mn, 1u);
          tc_mma_tf32_ta(t_dq, t_s + ao, dm_hi + bo, idesc_mn, 1u);
        }
        tc_commit(bar(E_FREE + st));
        if (j == nkb - 1) tc_commit(bar(E_DQFULL));
      }
    }
  } else if (warp < 6) {
    // ------------------------------------------------------------------ compute warps ---
    const int qd = warp & 3;
    const int row = 32 * qd + lane;
    const int64_t gi = i0 + row;
    const bool live = gi < D.Lq;
    const uint32_t t_row = tmem_base + ((uint32_t)(32 * qd) << 16);
    // Q and dO rows of this thread into tensor memory: the raw value is the hi operand, lo = x - tf32(x)
    {
      const float* src[2] = {q + (b * D.Lq + gi) * D.E + (int64_t)h * HD, dout + (b * D.Lq + gi) * D.Ev + (int64_t)h * HD};
#pragma unroll
      for (int w = 0; w < 2; ++w) {
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          uint32_t hi[32], lo[32];
#pragma unroll
          for (int c4 = 0; c4 < 8; ++c4) {
            float4 x = make_float4(0.f, 0.f, 0.f, 0.f);
            if (live) x = __ldg((const float4*)(src[w] + 32 * half + 4 * c4));
            hi[4 * c4] = __float_as_uint(x.x); hi[4 * c4 + 1] = __float_as_uint(x.y);
            hi[4 * c4 + 2] = __float_as_uint(x.z); hi[4 * c4 + 3] = __float_as_uint(x.w);
            lo[4 * c4] = __float_as_uint(tf32_lo(x.x)); lo[4 * c4 + 1] = __float_as_uint(tf32_lo(x.y));
            lo[4 * c4 + 2] = __float_as_uint(tf32_lo(x.z)); lo[4 * c4 + 3] = __float_as_uint(tf32_lo(x.w));
          }
          tc_st_32x32b_x32(t_row + (uint32_t)(128 * w + 32 * half), hi);
          tc_st_32x32b_x32(t_row + (uint32_t)(128 * w + 64 + 32 * half), lo);
        }
      }
      tc_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(E_QREADY));
    }
    const float l2 = live ? lse[(b * D.H + h) * D.Lq + gi] * 1.4426950408889634f : INFINITY;   // a dead row gets P = 0
    const float dl = live ? dlt[(b * D.H + h) * D.Lq + gi] : 0.0f;
    bool ok = true;
    for (int j = 0; j < nkb && ok; ++j) {
      const int64_t j0 = (int64_t)j * KT;
      ok = mbar_wait(bar(E_SFULL), (uint32_t)j & 1u, s_abort);
      if (!ok) break;
      tc_fence_after();
      int64_t lim = D.Lk - j0;
      if (D.causal && gi - j0 + 1 < lim) lim = gi - j0 + 1;
      const int nvalid = lim < 0 ? 0 : (lim > KT ? KT : (int)lim);
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        uint32_t sv[32], dp[32];
        tc_ld_32x32b_x32(t_row + 256u + (uint32_t)(32 * half), sv);
        tc_ld_32x32b_x32(t_row + 384u + (uint32_t)(32 * half), dp);
        tc_wait_ld();
#pragma unroll
        for (int c = 0; c < 32; ++c) {
          float p = fast_exp2(fmaf(__uint_as_float(sv[c]), D.scale_log2, -l2));
          if (c + 32 * half >= nvalid) p = 0.0f;
          const float ds = p * (__uint_as_float(dp[c]) - dl);
          sv[c] = __float_as_uint(ds);
          dp[c] = __float_as_uint(tf32_lo(ds));
        }
        tc_st_32x32b_x32(t_row + 256u + (uint32_t)(32 * half), sv);
        tc_st_32x32b_x32(t_row + 320u + (uint32_t)(32 * half), dp);
      }
      tc_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(E_DSREADY));
    }
    if (ok) ok = mbar_wait(bar(E_DQFULL), 0u, s_abort);
    if (ok) {
      tc_fence_after();
      uint32_t r0[32], r1[32];
      tc_ld_32x32b_x32(t_row + 448u, r0);
      tc_ld_32x32b_x32(t_row + 480u, r1);
      tc_wait_ld();
      if (live) {
        float* drow = dq + (b * D.Lq + gi) * D.E + (int64_t)h * HD;
#pragma unroll
        for (int c = 0; c < 32; c += 4) {
          *(float4*)(drow + c) = make_float4(__uint_as_float(r0[c]) * D.scale, __uint_as_float(r0[c + 1]) * D.scale,
                                             __uint_as_float(r0[c + 2]) * D.scale, __uint_as_float(r0[c + 3]) * D.scale);
          *(float4*)(drow + 32 + c) = make_float4(__uint_as_float(r1[c]) * D.scale, __uint_as_float(r1[c + 1]) * D.scale,
                                                  __uint_as_float(r1[c + 2]) * D.scale, __uint_as_float(r1[c + 3]) * D.scale);
        }
      }
    }
  } else {
    // --------------------------------------------- split warps: lo = x - tf32(x) twins ---
    const int tt = (warp - 6) * 32 + lane;
    bool ok = true;
    for (int j = 0; j < nkb && ok; ++j) {
      const int st = j & 1;
      ok = mbar_wait(bar(E_FULL + st), par(j), s_abort);
      if (!ok) break;
#pragma unroll
      for (int tile = 0; tile < 3; ++tile) {
        const float4* hi = (const float4*)(smem + st * DQ_STAGE_BYTES + tile * 32768);
        float4* lo = (float4*)(smem + st * DQ_STAGE_BYTES + tile * 32768 + 16384);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          float4 v = hi[tt + i * 128];
          v.x = tf32_lo(v.x); v.y = tf32_lo(v.y); v.z = tf32_lo(v.z); v.w = tf32_lo(v.w);
          lo[tt + i * 128] = v;
        }
      }
      fence_proxy_async();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(E_READY + st));
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
  }
  if (threadIdx.x == 0 && *s_abort != 0) atomicExch(dev_err, 4003);
}

// ------------------------------------------------------------------------------------------------------------------
// dK and dV of the attention backward pass on the tensor cores, in transposed form so that keys are the rows
// (TMEM lanes) of every accumulator.  One CTA owns 128 keys of one (batch, head): K lives in tensor memory (A operand),
// V in shared memory (A operand, K-major).  For every block of 64 queries:
//   S' = K Q'  and  dP' = V dO'    (B operands: the Q and dO tiles, K-major)
//   P' = exp(S' / sqrt(d) - lse_q),  dS' = P' (dP' - delta_q)     (compute warps; back through tensor memory)
//   dV += P' dO  and  dK += dS' Q   (B operands: the same Q and dO tiles loaded a second time MN-major, queries
//                                    being their K rows)
// A tile's shared memory is reloaded as soon as the MMAs that read it have completed, so the loads of the next block
// overlap the rest of the current one.  dK and dV accumulate in tensor memory over at most 32 query blocks.
//   TMEM columns: K hi 0, K lo 64, S' -> P' hi 128, P' lo 192, dP' -> dS' hi 256, dS' lo 320, dV 384, dK 448
constexpr int KV_VHI = 0, KV_VLO = 32768;                       // 4 chunks x [128 keys][16 floats]
constexpr int KV_QK = 65536, KV_DOK = 98304, KV_DOM = 131072, KV_QM = 163840;   // 64-query tiles: hi 16 KB + lo 16 KB each
constexpr int KV_ROWV = 196608;                                 // lse * log2(e) and delta of the block's 64 queries, two sets
constexpr int KV_BAR = KV_ROWV + 1024;
constexpr int KV_SMEM = KV_BAR + 256 + 1024;
constexpr int KV_MAX_BLOCKS = 32;
enum { F_KREADY = 0, F_VFULL, F_VREADY, F_FULL, F_READY = F_FULL + 4, F_FREE = F_READY + 4, F_SFULL = F_FREE + 4, F_PREADY, F_DONE, F_COUNT };

__global__ void __launch_bounds__(ATC_THREADS, 1)
attn_bwd_dkdv_tc_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmQmn,
                        const __grid_constant__ CUtensorMap tmDO, const __grid_constant__ CUtensorMap tmDOmn,
                        const __grid_constant__ CUtensorMap tmV, const float* __restrict__ k, const float* __restrict__ lse,
                        const float* __restrict__ dlt, float* __restrict__ dk, float* __restrict__ dv, AtcDims D,
                        int32_t* __restrict__ dev_err) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const uint32_t sb = smem_u32(smem);
  const uint32_t bar0 = sb + KV_BAR;
  auto bar = [&](int i) { return bar0 + 8u * (uint32_t)i; };
  volatile uint32_t* s_tmem = (volatile uint32_t*)(smem + KV_BAR + 8 * F_COUNT);
  volatile int* s_abort = (volatile int*)(smem + KV_BAR + 8 * F_COUNT + 8);
  volatile int* s_skip = (volatile int*)(smem + KV_BAR + 8 * F_COUNT + 16);
  float* rowv = (float*)(smem + KV_ROWV);   // [set][0: lse * log2e, 1: delta][64]

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t j0 = (int64_t)blockIdx.x * QT;   // first key of this CTA
  const int h = blockIdx.y;
  const int64_t b = blockIdx.z;
  // query blocks that see these keys: all of them, or under a causal mask those from the diagonal on
  const int ib0 = D.causal ? (int)(j0 / KT) : 0;
  const int nqb = (int)((D.Lq + KT - 1) / KT) - ib0;   // may be <= 0: nothing attends to these keys

  if (threadIdx.x == 0) {
    mbar_init(bar(F_KREADY), 4);
    mbar_init(bar(F_VFULL), 1);
    mbar_init(bar(F_VREADY), 4);
    for (int t = 0; t < 4; ++t) {
      mbar_init(bar(F_FULL + t), 1);
      mbar_init(bar(F_READY + t), 4);
      mbar_init(bar(F_FREE + t), 1);
    }
    mbar_init(bar(F_SFULL), 1);
    mbar_init(bar(F_PREADY), 4);
    mbar_init(bar(F_DONE), 1);
    *s_abort = 0;
    *s_skip = (*(volatile int32_t*)dev_err != 0) ? 1 : 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    fence_proxy_async();
  }
  __syncthreads();
  if (*s_skip != 0) return;
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32((const void*)s_tmem)), "r"(512u)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *s_tmem;
  // tile order: 0 = Q k-major, 1 = dO k-major, 2 = dO mn-major, 3 = Q mn-major
  const int tile_off[4] = {KV_QK, KV_DOK, KV_DOM, KV_QM};

  if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer ---
    if (lane == 0 && nqb > 0) {
      mbar_arrive_expect_tx(bar(F_VFULL), 32768u);
#pragma unroll
      for (int c = 0; c < 4; ++c) tma_load_2d(sb + KV_VHI + c * 8192, &tmV, h * HD + 16 * c, (int)(b * D.Lk + j0), bar(F_VFULL));
      bool ok = true;
      for (int i = 0; i < nqb && ok; ++i) {
        const int qrow = (int)(b * D.Lq + (int64_t)(ib0 + i) * KT);
        const uint32_t ph = (uint32_t)(i - 1) & 1u;
#pragma unroll
        for (int t = 0; t < 4; ++t) {
          if (i > 0 && !mbar_wait(bar(F_FREE + t), ph, s_abort)) { ok = false; break; }
          mbar_arrive_expect_tx(bar(F_FULL + t), 16384u);
          const uint32_t dst = sb + (uint32_t)tile_off[t];
          if (t == 0) {
            for (int c = 0; c < 4; ++c) tma_load_2d(dst + c * 4096, &tmQ, h * HD + 16 * c, qrow, bar(F_FULL + t));
          } else if (t == 1) {
            for (int c = 0; c < 4; ++c) tma_load_2d(dst + c * 4096, &tmDO, h * HD + 16 * c, qrow, bar(F_FULL + t));
          } else if (t == 2) {
            tma_load_3d(dst, &tmDOmn, 0, qrow, 2 * h, bar(F_FULL + t));
          } else {
            tma_load_3d(dst, &tmQmn, 0, qrow, 2 * h, bar(F_FULL + t));
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer ---
    if (lane == 0 && nqb > 0) {
      const uint32_t idesc_kk = (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(KT >> 3) << 17) | ((uint32_t)(QT >> 4) << 24);
      const uint32_t idesc_mn = idesc_kk | (1u << 16);
      const uint32_t t_k = tmem_base, t_p = tmem_base + 128u, t_ds = tmem_base + 256u, t_dv = tmem_base + 384u, t_dk = tmem_base + 448u;
      const uint64_t dv_hi = make_smem_desc(sb + KV_VHI, 16, 512, LAYOUT_SW64), dv_lo = make_smem_desc(sb + KV_VLO, 16, 512, LAYOUT_SW64);
      const uint64_t dqk_hi = make_smem_desc(sb + KV_QK, 16, 512, LAYOUT_SW64), dqk_lo = make_smem_desc(sb + KV_QK + 16384, 16, 512, LAYOUT_SW64);
      const uint64_t dok_hi = make_smem_desc(sb + KV_DOK, 16, 512, LAYOUT_SW64), dok_lo = make_smem_desc(sb + KV_DOK + 16384, 16, 512, LAYOUT_SW64);
      const uint64_t dom_hi = make_smem_desc(sb + KV_DOM, KT * 128, 512, LAYOUT_SW128_32B), dom_lo = make_smem_desc(sb + KV_DOM + 16384, KT * 128, 512, LAYOUT_SW128_32B);
      const uint64_t dqm_hi = make_smem_desc(sb + KV_QM, KT * 128, 512, LAYOUT_SW128_32B), dqm_lo = make_smem_desc(sb + KV_QM + 16384, KT * 128, 512, LAYOUT_SW128_32B);
      bool ok = mbar_wait(bar(F_KREADY), 0u, s_abort) && mbar_wait(bar(F_VREADY), 0u, s_abort);
      for (int i = 0; i < nqb && ok; ++i) {
        const uint32_t ph = (uint32_t)i & 1u;
        ok = mbar_wait(bar(F_READY + 0), ph, s_abort) && mbar_wait(bar(F_READY + 1), ph, s_abort);
        if (!ok) break;
        tc_fence_after();
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {   // S' = K Q' over the 64 features
          const uint64_t bo = (uint64_t)(((ks >> 1) * 4096 + (ks & 1) * 32) >> 4);
          const uint32_t ao = (uint32_t)(8 * ks);
          tc_mma_tf32_ta(t_p, t_k + 64u + ao, dqk_hi + bo, idesc_kk, ks > 0 ? 1u : 0u);
          tc_mma_tf32_ta(t_p, t_k + ao, dqk_lo + bo, idesc_kk, 1u);
          tc_mma_tf32_ta(t_p, t_k + ao, dqk_hi + bo, idesc_kk, 1u);
        }
        tc_commit(bar(F_FREE + 0));
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {   // dP' = V dO' over the 64 value features (A = V from shared memory)
          const uint64_t ao = (uint64_t)(((ks >> 1) * 8192 + (ks & 1) * 32) >> 4), bo = (uint64_t)(((ks >> 1) * 4096 + (ks & 1) * 32) >> 4);
          tc_mma_tf32(t_ds, dv_lo + ao, dok_hi + bo, idesc_kk, ks > 0 ? 1u : 0u);
          tc_mma_tf32(t_ds, dv_hi + ao, dok_lo + bo, idesc_kk, 1u);
          tc_mma_tf32(t_ds, dv_hi + ao, dok_hi + bo, idesc_kk, 1u);
        }
        tc_commit(bar(F_FREE + 1));
        tc_commit(bar(F_SFULL));
        ok = mbar_wait(bar(F_PREADY), ph, s_abort) && mbar_wait(bar(F_READY + 2), ph, s_abort) && mbar_wait(bar(F_READY + 3), ph, s_abort);
        if (!ok) break;
        tc_fence_after();
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {   // dV += P' dO over the 64 queries
          const uint64_t bo = (uint64_t)((ks * 1024) >> 4);
          const uint32_t ao = (uint32_t)(8 * ks);
          tc_mma_tf32_ta(t_dv, t_p + 64u + ao, dom_hi + bo, idesc_mn, (i > 0 || ks > 0) ? 1u : 0u);
          tc_mma_tf32_ta(t_dv, t_p + ao, dom_lo + bo, idesc_mn, 1u);
          tc_mma_tf32_ta(t_dv, t_p + ao, dom_hi + bo, idesc_mn, 1u);
        }
        tc_commit(bar(F_FREE + 2));
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {   // dK += dS' Q over the 64 queries
          const uint64_t bo = (uint64_t)((ks * 1024) >> 4);
          const uint32_t ao = (uint32_t)(8 * ks);
          tc_mma_tf32_ta(t_dk, t_ds + 64u + ao, dqm_hi + bo, idesc_mn, (i > 0 || ks > 0) ? 1u : 0u);
          tc_mma_tf32_ta(t_dk, t_ds + ao, dqm_lo + bo, idesc_mn, 1u);
          tc_mma_tf32_ta(t_dk, t_ds + ao, dqm_hi + bo, idesc_mn, 1u);
        }
        tc_commit(bar(F_FREE + 3));
        if (i == nqb - 1) tc_commit(bar(F_DONE));
      }
    }
  } else if (warp < 6) {
    // ------------------------------------------------------------------ compute warps ---
    const int qd = warp & 3;
    const int row = 32 * qd + lane;
    const int64_t kj = j0 + row;             // this thread's key
    const bool live = kj < D.Lk;
    const uint32_t t_row = tmem_base + ((uint32_t)(32 * qd) << 16);
    if (nqb > 0) {
      // K row of this thread into tensor memory: the raw value is the hi operand, lo = x - tf32(x)
      const float* src = k + (b * D.Lk + kj) * D.E + (int64_t)h * HD;
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        uint32_t hi[32], lo[32];
#pragma unroll
        for (int c4 = 0; c4 < 8; ++c4) {
          float4 x = make_float4(0.f, 0.f, 0.f, 0.f);
          if (live) x = __ldg((const float4*)(src + 32 * half + 4 * c4));
          hi[4 * c4] = __float_as_uint(x.x); hi[4 * c4 + 1] = __float_as_uint(x.y);
          hi[4 * c4 + 2] = __float_as_uint(x.z); hi[4 * c4 + 3] = __float_as_uint(x.w);
          lo[4 * c4] = __float_as_uint(tf32_lo(x.x)); lo[4 * c4 + 1] = __float_as_uint(tf32_lo(x.y));
          lo[4 * c4 + 2] = __float_as_uint(tf32_lo(x.z)); lo[4 * c4 + 3] = __float_as_uint(tf32_lo(x.w));
        }
        tc_st_32x32b_x32(t_row + (uint32_t)(32 * half), hi);
        tc_st_32x32b_x32(t_row + (uint32_t)(64 + 32 * half), lo);
      }
      tc_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(F_KREADY));
    }
    bool ok = true;
    for (int i = 0; i < nqb && ok; ++i) {
      const int64_t i0b = (int64_t)(ib0 + i) * KT;   // first query of the block
      const float* rv = rowv + (i & 1) * 128;
      ok = mbar_wait(bar(F_SFULL), (uint32_t)i & 1u, s_abort);
      if (!ok) break;
      tc_fence_after();
      // queries of the block this key is seen by: query < Lq (dead ones carry lse = +inf), and query >= key when causal
      int clo = 0;
      if (D.causal && kj - i0b > 0) clo = (kj - i0b) > KT ? KT : (int)(kj - i0b);
      if (!live) clo = KT;
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        uint32_t sv[32], dp[32], lo[32];
        tc_ld_32x32b_x32(t_row + 128u + (uint32_t)(32 * half), sv);
        tc_ld_32x32b_x32(t_row + 256u + (uint32_t)(32 * half), dp);
        tc_wait_ld();
#pragma unroll
        for (int c = 0; c < 32; ++c) {
          const int cq = c + 32 * half;
          float p = fast_exp2(fmaf(__uint_as_float(sv[c]), D.scale_log2, -rv[cq]));
          if (cq < clo) p = 0.0f;
          const float ds = p * (__uint_as_float(dp[c]) - rv[64 + cq]);
          sv[c] = __float_as_uint(p);
          lo[c] = __float_as_uint(tf32_lo(p));
          dp[c] = __float_as_uint(ds);
        }
        tc_st_32x32b_x32(t_row + 128u + (uint32_t)(32 * half), sv);
        tc_st_32x32b_x32(t_row + 192u + (uint32_t)(32 * half), lo);
#pragma unroll
        for (int c = 0; c < 32; ++c) lo[c] = __float_as_uint(tf32_lo(__uint_as_float(dp[c])));
        tc_st_32x32b_x32(t_row + 256u + (uint32_t)(32 * half), dp);
        tc_st_32x32b_x32(t_row + 320u + (uint32_t)(32 * half), lo);
      }
      tc_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(F_PREADY));
    }
    if (nqb > 0) {
      if (ok) ok = mbar_wait(bar(F_DONE), 0u, s_abort);
      if (ok) {
        tc_fence_after();
#pragma unroll
        for (int w = 0; w < 2; ++w) {   // 0: dV, 1: dK (scaled by 1 / sqrt(d))
          uint32_t r0[32], r1[32];
          tc_ld_32x32b_x32(t_row + 384u + (uint32_t)(64 * w), r0);
          tc_ld_32x32b_x32(t_row + 416u + (uint32_t)(64 * w), r1);
          tc_wait_ld();
          if (live) {
            const float sc = w == 0 ? 1.0f : D.scale;
            float* drow = (w == 0 ? dv + (b * D.Lk + kj) * D.Ev : dk + (b * D.Lk + kj) * D.E) + (int64_t)h * HD;
#pragma unroll
            for (int c = 0; c < 32; c += 4) {
              *(float4*)(drow + c) = make_float4(__uint_as_float(r0[c]) * sc, __uint_as_float(r0[c + 1]) * sc,
                                                 __uint_as_float(r0[c + 2]) * sc, __uint_as_float(r0[c + 3]) * sc);
              *(float4*)(drow + 32 + c) = make_float4(__uint_as_float(r1[c]) * sc, __uint_as_float(r1[c + 1]) * sc,
                                                      __uint_as_float(r1[c + 2]) * sc, __uint_as_float(r1[c + 3]) * sc);
            }
          }
        }
      }
    } else if (live) {
      // no query sees these keys: their gradients are zero
      float* r1 = dv + (b * D.Lk + kj) * D.Ev + (int64_t)h * HD;
      float* r2 = dk + (b * D.Lk + kj) * D.E + (int64_t)h * HD;
#pragma unroll
      for (int c = 0; c < HD; c += 4) {
        *(float4*)(r1 + c) = make_float4(0.f, 0.f, 0.f, 0.f);
        *(float4*)(r2 + c) = make_float4(0.f, 0.f, 0.f, 0.f);
      }
    }
  } else {
    // --------------------------------- split warps: lo twins, and the per-query lse / delta of each block ---
    const int tt = (warp - 6) * 32 + lane;
    auto split = [&](int off, int n16) {
      const float4* hi = (const float4*)(smem + off);
      float4* lo = (float4*)(smem + off + (n16 == 16 ? 32768 : 16384));
      for (int i = 0; i < n16; ++i) {
        float4 v = hi[tt + i * 128];
        v.x = tf32_lo(v.x); v.y = tf32_lo(v.y); v.z = tf32_lo(v.z); v.w = tf32_lo(v.w);
        lo[tt + i * 128] = v;
      }
    };
    bool ok = nqb > 0;
    if (ok) ok = mbar_wait(bar(F_VFULL), 0u, s_abort);
    if (ok) {
      split(KV_VHI, 16);
      fence_proxy_async();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(F_VREADY));
    }
    for (int i = 0; i < nqb && ok; ++i) {
      const uint32_t ph = (uint32_t)i & 1u;
      // lse * log2(e) and delta of the block's queries (set i & 1: the compute warps may still read the other set)
      if (tt < KT) {
        const int64_t gq = (int64_t)(ib0 + i) * KT + tt;
        float* rv = rowv + (i & 1) * 128;
        rv[tt] = gq < D.Lq ? lse[(b * D.H + h) * D.Lq + gq] * 1.4426950408889634f : INFINITY;
        rv[64 + tt] = gq < D.Lq ? dlt[(b * D.H + h) * D.Lq + gq] : 0.0f;
      }
#pragma unroll 1
      for (int t = 0; t < 4 && ok; ++t) {
        ok = mbar_wait(bar(F_FULL + t), ph, s_abort);
        if (!ok) break;
        split(tile_off[t], 8);
        fence_proxy_async();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar(F_READY + t));
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
  }
  if (threadIdx.x == 0 && *s_abort != 0) atomicExch(dev_err, 4004);
}

// FLUXB200_ATTN_TC = 0 keeps attention on the Float32 FMA kernels.
bool attn_tc_enabled() {
  static int on = -1;
  if (on < 0) {
    const char* e = getenv("FLUXB200_ATTN_TC");
    on = (e != nullptr && e[0] == '0') ? 0 : 1;
  }
  return on != 0;
}

// FLUXB200_ATTN_BWD_TC = 0 keeps the backward pass on the Float32 FMA kernels.
bool attn_bwd_tc_enabled() {
  static int on = -1;
  if (on < 0) {
    const char* e = getenv("FLUXB200_ATTN_BWD_TC");
    on = (e != nullptr && e[0] == '0') ? 0 : 1;
  }
  return on != 0;
}

// 3-d view {32, rows, cols / 32} of a row-major [rows][cols] matrix whose rows are the K dimension of an MN-major
// operand: box {32, box_rows, chunks}.
bool encode_rows3d(CUtensorMap* map, const float* base, int64_t rows, int64_t cols, uint32_t box_rows, uint32_t chunks) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn || cols % 32 != 0) return false;
  cuuint64_t gdim[3] = {32, (cuuint64_t)rows, (cuuint64_t)(cols / 32)};
  cuuint64_t gstride[2] = {(cuuint64_t)cols * sizeof(float), 128};
  cuuint32_t box[3] = {32, box_rows, chunks};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, (void*)base, gdim, gstride, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

}  // namespace

// Returns FB_ERR_UNSUPPORTED when the shape is not one this kernel takes (the caller then uses the FMA kernels).
int32_t fb_attn_fwd_tc(fb_ctx* ctx, cudaStream_t stream, const float* q, const float* k, const float* v, const uint8_t* mask,
                       float* o, float* lse, int64_t e_dim, int64_t ev_dim, int64_t lq, int64_t lk, int64_t batch, int nheads,
                       int causal) {
  if (!attn_tc_enabled() || mask != nullptr || nheads < 1) return FB_ERR_UNSUPPORTED;
  if (e_dim != (int64_t)nheads * HD || ev_dim != (int64_t)nheads * HD) return FB_ERR_UNSUPPORTED;
  if (lq < 1 || lk < 1 || batch < 1 || batch * lq > 0x7fffff00 || batch * lk > 0x7fffff00 || batch > 65535 || nheads > 65535)
    return FB_ERR_UNSUPPORTED;
  if (!fb_aligned16(q) || !fb_aligned16(k) || !fb_aligned16(v) || !fb_aligned16(o)) return FB_ERR_UNSUPPORTED;
  CUtensorMap tmK, tmV;
  if (!encode_map(&tmK, k, batch * lk, e_dim, e_dim, 16, KT, CU_TENSOR_MAP_SWIZZLE_64B) ||
      !encode_rows3d(&tmV, v, batch * lk, ev_dim, KT, HD / 32))
    return FB_ERR_UNSUPPORTED;
  AtcDims D;
  D.E = e_dim; D.Ev = ev_dim; D.Lq = lq; D.Lk = lk; D.H = nheads; D.causal = causal ? 1 : 0;
  D.scale = 1.0f / sqrtf((float)HD);
  D.scale_log2 = D.scale * 1.4426950408889634f;
  dim3 grid((unsigned)((lq + QT - 1) / QT), (unsigned)nheads, (unsigned)batch);
  FB_CUDA(cudaFuncSetAttribute(attn_fwd_tc2_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, ATC2_SMEM));
  attn_fwd_tc2_kernel<<<grid, ATC_THREADS, ATC2_SMEM, stream>>>(q, tmK, tmV, o, lse, D, ctx->dev_error);
  FB_LAUNCH_CHECK();
  return FB_OK;
}

// dQ of the backward pass; FB_ERR_UNSUPPORTED when the shape is not one this kernel takes.
int32_t fb_attn_bwd_dq_tc(fb_ctx* ctx, cudaStream_t stream, const float* q, const float* k, const float* v, const uint8_t* mask,
                          const float* lse, const float* dlt, const float* dout, float* dq, int64_t e_dim, int64_t ev_dim,
                          int64_t lq, int64_t lk, int64_t batch, int nheads, int causal) {
  if (!attn_tc_enabled() || !attn_bwd_tc_enabled() || mask != nullptr || nheads < 1) return FB_ERR_UNSUPPORTED;
  if (e_dim != (int64_t)nheads * HD || ev_dim != (int64_t)nheads * HD) return FB_ERR_UNSUPPORTED;
  if (lq < 1 || lk < 1 || batch < 1 || batch * lq > 0x7fffff00 || batch * lk > 0x7fffff00 || batch > 65535 || nheads > 65535)
    return FB_ERR_UNSUPPORTED;
  if ((lk + KT - 1) / KT > DQ_MAX_BLOCKS) return FB_ERR_UNSUPPORTED;   // dQ accumulates in tensor memory over <= 2048 keys
  if (!fb_aligned16(q) || !fb_aligned16(k) || !fb_aligned16(v) || !fb_aligned16(dout) || !fb_aligned16(dq)) return FB_ERR_UNSUPPORTED;
  CUtensorMap tmK, tmKmn, tmV;
  if (!encode_map(&tmK, k, batch * lk, e_dim, e_dim, 16, KT, CU_TENSOR_MAP_SWIZZLE_64B) ||
      !encode_rows3d(&tmKmn, k, batch * lk, e_dim, KT, HD / 32) ||
      !encode_map(&tmV, v, batch * lk, ev_dim, ev_dim, 16, KT, CU_TENSOR_MAP_SWIZZLE_64B))
    return FB_ERR_UNSUPPORTED;
  AtcDims D;
  D.E = e_dim; D.Ev = ev_dim; D.Lq = lq; D.Lk = lk; D.H = nheads; D.causal = causal ? 1 : 0;
  D.scale = 1.0f / sqrtf((float)HD);
  D.scale_log2 = D.scale * 1.4426950408889634f;
  FB_CUDA(cudaFuncSetAttribute(attn_bwd_dq_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, DQ_SMEM));
  dim3 grid((unsigned)((lq + QT - 1) / QT), (unsigned)nheads, (unsigned)batch);
  attn_bwd_dq_tc_kernel<<<grid, ATC_THREADS, DQ_SMEM, stream>>>(tmK, tmKmn, tmV, q, dout, lse, dlt, dq, D, ctx->dev_error);
  FB_LAUNCH_CHECK();
  return FB_OK;
}

// dK and dV of the backward pass; FB_ERR_UNSUPPORTED when the shape is not one this kernel takes.
int32_t fb_attn_bwd_dkdv_tc(fb_ctx* ctx, cudaStream_t stream, const float* q, const float* k, const float* v, const uint8_t* mask,
                            const float* lse, const float* dlt, const float* dout, float* dk, float* dv, int64_t e_dim,
                            int64_t ev_dim, int64_t lq, int64_t lk, int64_t batch, int nheads, int causal) {
  if (!attn_tc_enabled() || !attn_bwd_tc_enabled() || mask != nullptr || nheads < 1) return FB_ERR_UNSUPPORTED;
  if (e_dim != (int64_t)nheads * HD || ev_dim != (int64_t)nheads * HD) return FB_ERR_UNSUPPORTED;
  if (lq < 1 || lk < 1 || batch < 1 || batch * lq > 0x7fffff00 || batch * lk > 0x7fffff00 || batch > 65535 || nheads > 65535)
    return FB_ERR_UNSUPPORTED;
  if ((lq + KT - 1) / KT > KV_MAX_BLOCKS) return FB_ERR_UNSUPPORTED;   // accumulation in tensor memory over <= 2048 queries
  if (!fb_aligned16(q) || !fb_aligned16(k) || !fb_aligned16(v) || !fb_aligned16(dout) || !fb_aligned16(dk) || !fb_aligned16(dv))
    return FB_ERR_UNSUPPORTED;
  CUtensorMap tmQ, tmQmn, tmDO, tmDOmn, tmV;
  if (!encode_map(&tmQ, q, batch * lq, e_dim, e_dim, 16, KT, CU_TENSOR_MAP_SWIZZLE_64B) ||
      !encode_rows3d(&tmQmn, q, batch * lq, e_dim, KT, HD / 32) ||
      !encode_map(&tmDO, dout, batch * lq, ev_dim, ev_dim, 16, KT, CU_TENSOR_MAP_SWIZZLE_64B) ||
      !encode_rows3d(&tmDOmn, dout, batch * lq, ev_dim, KT, HD / 32) ||
      !encode_map(&tmV, v, batch * lk, ev_dim, ev_dim, 16, QT, CU_TENSOR_MAP_SWIZZLE_64B))
    return FB_ERR_UNSUPPORTED;
  AtcDims D;
  D.E = e_dim; D.Ev = ev_dim; D.Lq = lq; D.Lk = lk; D.H = nheads; D.causal = causal ? 1 : 0;
  D.scale = 1.0f / sqrtf((float)HD);
  D.scale_log2 = D.scale * 1.4426950408889634f;
  FB_CUDA(cudaFuncSetAttribute(attn_bwd_dkdv_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, KV_SMEM));
  dim3 grid((unsigned)((lk + QT - 1) / QT), (unsigned)nheads, (unsigned)batch);
  attn_bwd_dkdv_tc_kernel<<<grid, ATC_THREADS, KV_SMEM, stream>>>(tmQ, tmQmn, tmDO, tmDOmn, tmV, k, lse, dlt, dk, dv, D,
                                                                   ctx->dev_error);
  FB_LAUNCH_CHECK();
  return FB_OK;
}
