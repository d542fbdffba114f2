// The attention core of absorbed MLA decode on the 5th-generation tensor cores (tcgen05, accumulators in tensor
// memory): one pass over the bf16 latent cache with an online softmax, split over the sequence (flash-decoding).
// Replaces attn_tile_score_k / max / sum / accum (src/kimi_exec.cu:414-475) and the three-pass tiled_attention
// (:692-716).  Same interface and partial results as mla_attend_kernel (mla_attend.cu), which stays as the fallback.
//
// All 64 heads of a sequence share one latent row per token: per token 1,152 bytes are read once from HBM and feed
// 64 x (576 + 512) multiply-adds.  A CTA owns one (sequence, token range) and walks it in tiles of 64 tokens:
//
//   S [heads x tokens]     = Q [heads x 576] . C^T          36 MMAs M128 N64 K16: A = Q (shared memory, K-major; rows
//                                                            64..127 of the M = 128 shape address whatever follows Q and
//                                                            are never read back), B = the tile (K-major)
//   P = exp2(S * scale * log2 e - m)                         one head row per thread (tcgen05.ld), bf16, to shared memory
//   O^T [latent x heads]  += C^T [latent x tokens] . P^T     16 MMAs M128 N64 K16: A = the SAME tile bytes read MN-major
//                                                            (four blocks of 128 latent columns), B = P (K-major)
//
// The tile lies in shared memory in 8 x 16-byte core matrices without swizzle: element (token t, column c) at
// (c / 8) * 1040 + (t / 8) * 128 + (t % 8) * 16 + (c % 8) * 2.  Read K-major that is a [64 tokens x 576] operand, read
// MN-major the same bytes are a [512 x 64 tokens] operand: one copy from HBM serves both products.
//
// The running maximum is kept lazily: a head's reference m changes only when a tile's maximum exceeds it by more than
// 40 (natural units); then all four warps of the consumer group rescale O^T in tensor memory.  exp(s - m) stays far
// inside fp32 and bf16 range meanwhile, and the merge over the splits needs a consistent (m, sum, O) only.
//
// Warps: 0..3 consumers (0 and 1 own the 64 head rows of S; all four own the 128 lanes of O^T), 4..7 producers (two per
// tile buffer, 16-byte cp.async in an order that is coalesced in HBM and conflict-free in shared memory), 8: one lane
// issues the MMAs.  Every mbarrier wait is bounded; on a timeout the CTA records an error, still releases its tensor
// memory and returns.
#include "common.cuh"
#include "tmem_io.cuh"

namespace blok {

constexpr int kTaHeads = 64, kTaD = 576, kTaDV = 512;
constexpr int kTaTile = 64;                              // tokens per tile
constexpr int kTaKG = kTaD / 8;                          // 16-byte column groups of a cache row
constexpr int kTaLbo = kTaTile * 16;                     // bytes between column groups (tile, Q and P alike: 64 rows)
constexpr int kTaSbo = 128;                              // bytes between 8-row groups
constexpr int kTaTLbo = kTaLbo + 16;                     // the tile's column groups: + 16 bytes, so that a row's 8 neighbouring
                                                         // groups, copied by 8 neighbouring lanes, land in 8 different banks
constexpr int kTaTileBytes = kTaKG * kTaTLbo;            // 74,880
constexpr int kTaQBytes = kTaKG * kTaLbo;                // 64 head rows
constexpr int kTaPBytes = (kTaTile / 8) * kTaLbo;        // P: [64 heads x 64 tokens] bf16, K (token) major
constexpr int kTaSmemBytes = kTaQBytes + 2 * kTaTileBytes + kTaPBytes;
constexpr int kTaConsumers = 128, kTaProducers = 128;
constexpr int kTaThreads = kTaConsumers + kTaProducers + 32;
constexpr int kTaTmemCols = 512;                         // S: 2 x 64 columns, O^T: 4 x 64 columns
constexpr int kTaColO = 128;
constexpr unsigned kTaSpinLimit = 1u << 21;
constexpr float kTaLazy = 57.7f;                         // 40 natural units in the log2 domain
constexpr int kTaTraceTiles = 64;
// The score product as M = 64 (the 64 heads, no idle rows): its accumulator rows 16 w .. 16 w + 15 lie in lanes 0..15 of
// warp w's quarter of tensor memory, so all four consumer warps take 16 head rows each.  false: M = 128 with 64 idle
// rows, head h in lane h, two softmax warps.
#ifndef BLOK_MLA_TC_M64
#define BLOK_MLA_TC_M64 1
#endif
constexpr bool kTaM64 = BLOK_MLA_TC_M64 != 0;
constexpr int kTaSoftmaxWarps = kTaM64 ? 4 : 2;

__device__ __forceinline__ float ta_ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// bf16 pair (hi in the upper half), both rounded to nearest even
__device__ __forceinline__ uint32_t ta_pack_bf16x2(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}

__device__ unsigned g_mla_tc_error = 0;

__device__ __forceinline__ void ta_cp16(uint32_t dst, const void *src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void ta_cp16_zfill(uint32_t dst, const void *src, uint32_t src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
// Shared-memory matrix descriptor without swizzle: start address, leading and stride byte offsets (16-byte units),
// descriptor version 1.  K-major operand: leading = between column groups along K, stride = between 8-row groups.
// MN-major operand: leading = between 8-groups along K, stride = between 8-element groups along M / N.
__device__ __forceinline__ uint64_t ta_desc(uint32_t saddr, uint32_t lbo, uint32_t sbo) {
  return (uint64_t)((saddr & 0x3FFFFu) >> 4) | ((uint64_t)(lbo >> 4) << 16) | ((uint64_t)(sbo >> 4) << 32) | (1ull << 46);
}
__device__ __forceinline__ void ta_mma(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
      "}\n" ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void ta_commit(uint32_t mbar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(mbar) : "memory");
}
__device__ __forceinline__ void ta_arrive(uint32_t mbar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(mbar) : "memory");
}
__device__ __forceinline__ bool ta_test(uint32_t mbar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t"
      "}\n"
      : "=r"(ok)
      : "r"(mbar), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait for the given phase parity; false (and the error word set) on a timeout.
__device__ __forceinline__ bool ta_wait(uint32_t mbar, uint32_t parity, unsigned code) {
  for (unsigned it = 0; it < kTaSpinLimit; ++it) {
    uint32_t ok;
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t"
        "}\n"
        : "=r"(ok)
        : "r"(mbar), "r"(parity)
        : "memory");
    if (ok) return true;
    __nanosleep(64);
  }
  atomicExch(&g_mla_tc_error, code);
  return false;
}
// Barrier of the 128 consumer threads that also ORs their failure flags: after a timeout all of them leave together.
__device__ __forceinline__ bool ta_consumers_sync(bool failed) {
  uint32_t any;
  asm volatile(
      "{\n\t"
      ".reg .pred p, q;\n\t"
      "setp.ne.u32 q, %1, 0;\n\t"
      "bar.red.or.pred p, 1, %2, q;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t"
      "}\n"
      : "=r"(any)
      : "r"((uint32_t)failed), "n"(kTaConsumers)
      : "memory");
  return any != 0;
}

size_t mla_attend_tc_smem_bytes() { return kTaSmemBytes; }

// grid = (splits, B); arguments as mla_attend_kernel.  PAGED: page_rows is a multiple of the 64-token tile.
template <bool PAGED>
__global__ void __launch_bounds__(kTaThreads, 1)
    mla_attend_tc_kernel(const uint16_t *__restrict__ q, const uint16_t *__restrict__ cache, long ctx_stride,
                         const int *__restrict__ seq_len, float scale, float *__restrict__ part_o, float *__restrict__ part_ml,
                         const int *__restrict__ block_table, const int *__restrict__ slot_of, int table_stride, int page_rows,
                         long long *__restrict__ trace) {
  extern __shared__ __align__(128) unsigned char smem[];
  __shared__ __align__(8) unsigned long long s_bar[9];
  __shared__ uint32_t s_tmem;
  __shared__ float s_alpha[kTaHeads];
  __shared__ int s_need[2][4];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int split = blockIdx.x, splits = gridDim.x, b = blockIdx.y;
  const int seq = seq_len[b];
  const int ntiles = (seq + kTaTile - 1) / kTaTile;
  const int per = (ntiles + splits - 1) / splits;
  const int ts = split * per, te = min(ntiles, ts + per);
  float *my_ml = part_ml + ((size_t)b * splits + split) * kTaHeads * 2;
  if (ts >= te) {  // nothing to do for this split: mark it empty for the merge
    if (tid < kTaHeads) {
      my_ml[tid * 2] = -INFINITY;
      my_ml[tid * 2 + 1] = 0.f;
    }
    return;
  }
  const int nt = te - ts;
  const uint32_t sQ = (uint32_t)__cvta_generic_to_shared(smem);
  const uint32_t sT = sQ + kTaQBytes;
  const uint32_t sP = sT + 2 * kTaTileBytes;
  unsigned char *Pp = smem + kTaQBytes + 2 * kTaTileBytes;
  const uint32_t bar0 = (uint32_t)__cvta_generic_to_shared(&s_bar[0]);
  // full[buf]: the buffer's two producer warps; sfull[buf]: the S MMAs' commit; sfree[buf]: the two softmax warps have
  // read S; pfull: they have written P; empty[buf]: the commit behind the tile's P.C MMAs (tile buffer and P are free)
  const uint32_t bar_full = bar0, bar_sfull = bar0 + 16, bar_sfree = bar0 + 32, bar_pfull = bar0 + 48, bar_empty = bar0 + 56;
  if (tid == 0) {
    for (int i = 0; i < 2; ++i) {
      asm volatile("mbarrier.init.shared::cta.b64 [%0], 2;" ::"r"(bar_full + 8 * i) : "memory");
      asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(bar_sfull + 8 * i) : "memory");
      asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar_sfree + 8 * i), "r"(kTaSoftmaxWarps) : "memory");
      asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(bar_empty + 8 * i) : "memory");
    }
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar_pfull), "r"(kTaSoftmaxWarps) : "memory");
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"((uint32_t)__cvta_generic_to_shared(&s_tmem)),
                 "r"((uint32_t)kTaTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  {
    // Q [64 heads x 576] into the core-matrix layout: consecutive threads take consecutive heads of one column group
    const uint16_t *qb = q + (size_t)b * kTaHeads * kTaD;
    for (int u = tid; u < kTaHeads * kTaKG; u += kTaThreads) {
      const int kg = u >> 6, h = u & 63;
      ta_cp16(sQ + kg * kTaLbo + h * 16, qb + (size_t)h * kTaD + kg * 8);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = s_tmem;
  bool failed = false;
  // diagnostics (trace != NULL): CTA (0, 0) stamps, per tile, [0] buffer free, [1] tile landed, [2] S issued,
  // [3] S seen by the softmax warps, [4] P handed over, [5] P.C issued (nanoseconds)
  auto stamp = [&](int n, int slot) {
    if (trace && blockIdx.x == 0 && blockIdx.y == 0 && n < kTaTraceTiles) {
      long long t;
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
      trace[n * 16 + slot] = t;
    }
  };

  if (warp >= 4 && warp < 8) {
    // ---- producers: warps 4, 5 fill buffer 0 with the even tiles, warps 6, 7 buffer 1 with the odd ones ----
    const int buf = (warp - 4) >> 1, wi = (warp - 4) & 1;
    const uint16_t *cache_b = PAGED ? cache : cache + (size_t)b * ctx_stride * kTaD;
    const int *table_b = PAGED ? block_table + (size_t)(slot_of ? slot_of[b] : b) * table_stride : nullptr;
    const int g8 = lane & 7, t4 = lane >> 3;
    for (int n = buf; n < nt; n += 2) {
      if (n >= 2 && !ta_wait(bar_empty + 8 * buf, (uint32_t)(((n >> 1) - 1) & 1), 1u)) {
        failed = true;
        break;
      }
      if (wi == 0 && lane == 0) stamp(n, 0);
      const int tok0 = (ts + n) * kTaTile;
      const uint16_t *base = cache_b;
      int first = 0;  // the row of `base` that holds token 0
      if (PAGED) {
        base = cache + (size_t)table_b[tok0 / page_rows] * page_rows * kTaD;
        first = tok0 % page_rows - tok0;
      }
      // a warp's copy: 4 tokens x 8 column groups = 128 contiguous bytes (a whole line) of each of 4 rows in HBM; the
      // 32 pieces fall into the 8 bank groups of shared memory four times each
      const uint32_t dst0 = sT + buf * kTaTileBytes + g8 * kTaTLbo + t4 * 16;
      if (tok0 + kTaTile <= seq) {
        // a whole tile: every address is a constant offset from two per-tile bases, so the warp issues its 72 copies
        // back to back (one warp per scheduler has nobody to hide address arithmetic behind)
        const unsigned char *src0 = reinterpret_cast<const unsigned char *>(base + (size_t)(tok0 + first + t4) * kTaD) + g8 * 16;
#pragma unroll
        for (int i = 0; i < kTaTile / 8; ++i) {
          const unsigned char *sa = src0 + (size_t)(2 * i + wi) * 4 * kTaD * 2;  // tokens 8 i + 4 wi + t4
          const uint32_t da = dst0 + i * kTaSbo + wi * 64;
#pragma unroll
          for (int kb = 0; kb < kTaKG / 8; ++kb)
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(da + kb * 8 * kTaTLbo), "l"(sa + kb * 128));
        }
      } else {
#pragma unroll 2
        for (int i = 0; i < kTaTile / 8; ++i) {
          const int tok = tok0 + 8 * i + 4 * wi + t4;
          const int row = min(tok, seq - 1) + first;  // rows past the end are filled with zeros (their P is zero too)
          const uint16_t *sa = base + (size_t)row * kTaD + g8 * 8;
          const uint32_t da = dst0 + i * kTaSbo + wi * 64;
          for (int kb = 0; kb < kTaKG / 8; ++kb) ta_cp16_zfill(da + kb * 8 * kTaTLbo, sa + kb * 64, tok < seq ? 16u : 0u);
        }
      }
      asm volatile("cp.async.commit_group;" ::: "memory");
      if (wi == 0 && lane == 0 && n + 2 < nt) {
        // The buffer's next tile starts its way from HBM to L2 now: by the time the buffer is free again (this tile's
        // two products later) the copies above find it there, and HBM has been busy meanwhile.  A tile is contiguous
        // (dense cache, or inside a page); only rows of the sequence are touched.
        const int ptok = tok0 + 2 * kTaTile;
        const int prow = min(kTaTile, seq - ptok);
        const uint16_t *pbase = cache_b;
        int pfirst = 0;
        if (PAGED) {
          pbase = cache + (size_t)table_b[ptok / page_rows] * page_rows * kTaD;
          pfirst = ptok % page_rows - ptok;
        }
        asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(pbase + (size_t)(ptok + pfirst) * kTaD),
                     "r"((uint32_t)(prow * kTaD * 2))
                     : "memory");
      }
      if (wi == 0 && lane == 0) stamp(n, 6);
      asm volatile("cp.async.wait_group 0;" ::: "memory");
      if (wi == 0 && lane == 0) stamp(n, 7);
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // the tile is read by the tensor core's proxy
      __syncwarp();
      if (lane == 0) ta_arrive(bar_full + 8 * buf);
      if (wi == 0 && lane == 0) stamp(n, 1);
    }
  } else if (warp == 8) {
    if (lane == 0) {
      // ---- the MMA thread ----
      const uint32_t idesc_128 = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(kTaTile >> 3) << 17) | ((128u >> 4) << 24);
      const uint32_t idesc_s = kTaM64 ? (idesc_128 & ~(31u << 24)) | ((64u >> 4) << 24) : idesc_128;
      const uint32_t idesc_pv = idesc_128 | (1u << 15);  // A (the tile) MN-major
      const uint64_t q_desc = ta_desc(sQ, kTaLbo, kTaSbo);
      auto issue_s = [&](int n) {
        const int buf = n & 1;
        stamp(n, 12);
        const uint64_t c_desc = ta_desc(sT + buf * kTaTileBytes, kTaTLbo, kTaSbo);
#pragma unroll 4
        for (int kk = 0; kk < kTaD / 16; ++kk)
          ta_mma(tmem + 64 * buf, q_desc + (uint64_t)(kk * ((2 * kTaLbo) >> 4)), c_desc + (uint64_t)(kk * ((2 * kTaTLbo) >> 4)), idesc_s,
                 kk > 0 ? 1u : 0u);
        ta_commit(bar_sfull + 8 * buf);
        stamp(n, 2);
      };
      auto issue_pv = [&](int n) {
        const int buf = n & 1;
        stamp(n, 13);
        // block j: latent columns [128 j, +128) = column groups [16 j, +16); a K step is 16 tokens = two 8-row groups.
        // The four blocks take turns: consecutive MMAs then accumulate into different columns of tensor memory and do
        // not wait for one another.
        const uint64_t p_desc = ta_desc(sP, kTaLbo, kTaSbo);
#pragma unroll
        for (int kk = 0; kk < kTaTile / 16; ++kk) {
#pragma unroll
          for (int j = 0; j < kTaDV / 128; ++j) {
            const uint64_t a_desc = ta_desc(sT + buf * kTaTileBytes + j * 16 * kTaTLbo, kTaSbo, kTaTLbo);
            ta_mma(tmem + kTaColO + 64 * j, a_desc + (uint64_t)(kk * ((2 * kTaSbo) >> 4)), p_desc + (uint64_t)(kk * ((2 * kTaLbo) >> 4)),
                   idesc_pv, (n > 0 || kk > 0) ? 1u : 0u);
          }
        }
        ta_commit(bar_empty + 8 * buf);
        stamp(n, 5);
      };
      if (!ta_wait(bar_full, 0u, 2u)) failed = true;
      if (!failed) {
        tc_fence_after();
        issue_s(0);
      }
      for (int n = 0; n < nt && !failed; ++n) {
        // the next tile's scores go first when that tile has landed already: they run under this tile's softmax
        bool early = false;
        const int nn = n + 1, nb = nn & 1;
        if (nn < nt && ta_test(bar_full + 8 * nb, (uint32_t)((nn >> 1) & 1)) &&
            (nn < 2 || ta_test(bar_sfree + 8 * nb, (uint32_t)(((nn >> 1) - 1) & 1)))) {
          tc_fence_after();
          issue_s(nn);
          early = true;
        }
        if (!ta_wait(bar_pfull, (uint32_t)(n & 1), 3u)) {
          failed = true;
          break;
        }
        tc_fence_after();
        issue_pv(n);
        if (!early && nn < nt) {
          if (!ta_wait(bar_full + 8 * nb, (uint32_t)((nn >> 1) & 1), 4u) ||
              (nn >= 2 && !ta_wait(bar_sfree + 8 * nb, (uint32_t)(((nn >> 1) - 1) & 1), 5u))) {
            failed = true;
            break;
          }
          tc_fence_after();
          issue_s(nn);
        }
      }
    }
  } else {
    // ---- consumers ----
    const float sl2 = scale * 1.4426950408889634f;
    float m_ref = -INFINITY, l = 0.f;
    // this thread's head row of S (row_ok: the lane holds one)
    const bool row_ok = kTaM64 ? lane < 16 : true;
    const int head = kTaM64 ? 16 * warp + lane : tid;
    for (int n = 0; n < nt; ++n) {
      const int buf = n & 1;
      uint32_t pk[kTaTile / 2];
      if (warp < kTaSoftmaxWarps) {
        bool need = false;
        if (!failed && !ta_wait(bar_sfull + 8 * buf, (uint32_t)((n >> 1) & 1), 6u)) failed = true;
        if (!failed) {
          if (tid == 0) stamp(n, 3);
          tc_fence_after();
          uint32_t r[kTaTile];
          tmem_ld64(tmem + ((uint32_t)(32 * warp) << 16) + 64 * buf, r);
          tmem_wait_ld();
          if (tid == 0) stamp(n, 8);
          tc_fence_before();
          __syncwarp();
          if (lane == 0) ta_arrive(bar_sfree + 8 * buf);
          const int tok0 = (ts + n) * kTaTile;
          if (tok0 + kTaTile > seq) {  // the sequence's last tile: tokens past the end take no weight
#pragma unroll
            for (int j = 0; j < kTaTile; ++j)
              if (tok0 + j >= seq) r[j] = 0xff800000u;
          }
          float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
          for (int j = 0; j < kTaTile; j += 2) {
            mx0 = fmaxf(mx0, __uint_as_float(r[j]));
            mx1 = fmaxf(mx1, __uint_as_float(r[j + 1]));
          }
          const float mx = fmaxf(mx0, mx1) * sl2;  // the scale is positive
          float alpha = 1.f;
          if (n == 0) {
            m_ref = mx;  // the split's first tile holds at least one token
          } else if (mx > m_ref + kTaLazy) {
            alpha = exp2f(m_ref - mx);
            m_ref = mx;
            need = row_ok;
          }
          if (row_ok) s_alpha[head] = alpha;
          const float nm = -m_ref;
          float sum0 = 0.f, sum1 = 0.f;
#pragma unroll
          for (int j = 0; j < kTaTile; j += 2) {
            // the probabilities enter the second product rounded to bf16 (as the reference rounds them, :466); the
            // normaliser sums the same rounded values
            const uint32_t pp = ta_pack_bf16x2(ta_ex2(fmaf(__uint_as_float(r[j]), sl2, nm)), ta_ex2(fmaf(__uint_as_float(r[j + 1]), sl2, nm)));
            sum0 += __uint_as_float(pp << 16);
            sum1 += __uint_as_float(pp & 0xffff0000u);
            pk[j >> 1] = pp;
          }
          l = l * alpha + (sum0 + sum1);
          if (tid == 0) stamp(n, 9);
        }
        need = __any_sync(0xffffffffu, need);
        if (lane == 0) s_need[buf][warp] = need ? 1 : 0;
      }
      if (ta_consumers_sync(failed)) {
        failed = true;
        break;
      }
      if (s_need[buf][0] | s_need[buf][1] | (kTaM64 ? s_need[buf][2] | s_need[buf][3] : 0)) {
        // a head's reference maximum moved (never in tile 0): every lane of O^T scales its 4 x 64 head columns, once the
        // previous tile's MMAs have finished with them
        if (!ta_wait(bar_empty + 8 * ((n - 1) & 1), (uint32_t)(((n - 1) >> 1) & 1), 7u)) failed = true;
        if (!failed) {
          tc_fence_after();
#pragma unroll 1
          for (int j = 0; j < kTaDV / 128; ++j) {
            uint32_t o[64];
            const uint32_t ta = tmem + ((uint32_t)(32 * warp) << 16) + kTaColO + 64 * j;
            tmem_ld64(ta, o);
            tmem_wait_ld();
#pragma unroll
            for (int c = 0; c < 64; ++c) o[c] = __float_as_uint(__uint_as_float(o[c]) * s_alpha[c]);
            tmem_st64(ta, o);
          }
          tmem_wait_st();
          tc_fence_before();
        }
        if (ta_consumers_sync(failed)) {
          failed = true;
          break;
        }
      }
      if (tid == 0) stamp(n, 10);
      if (warp < kTaSoftmaxWarps && !failed) {
        if (n > 0 && !ta_wait(bar_empty + 8 * ((n - 1) & 1), (uint32_t)(((n - 1) >> 1) & 1), 8u)) {
          failed = true;  // reaches the others at the next tile's barrier
        } else {
          if (tid == 0) stamp(n, 11);
          if (row_ok) {
#pragma unroll
            for (int kg = 0; kg < kTaTile / 8; ++kg)
              *reinterpret_cast<uint4 *>(Pp + kg * kTaLbo + head * 16) = make_uint4(pk[4 * kg], pk[4 * kg + 1], pk[4 * kg + 2], pk[4 * kg + 3]);
          }
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
          __syncwarp();
          if (lane == 0) ta_arrive(bar_pfull);
          if (tid == 0) stamp(n, 4);
        }
      }
    }
    // ---- the split's partial result: O^T [latent lane x head column] -> part_o [head][512], (m, sum) per head ----
    if (!failed && !ta_wait(bar_empty + 8 * ((nt - 1) & 1), (uint32_t)(((nt - 1) >> 1) & 1), 9u)) failed = true;
    failed = ta_consumers_sync(failed);
    if (!failed) {
      tc_fence_after();
      float *po = part_o + ((size_t)b * splits + split) * kTaHeads * kTaDV;
#pragma unroll 1
      for (int j = 0; j < kTaDV / 128; ++j) {
#pragma unroll 1
        for (int half = 0; half < 2; ++half) {
          uint32_t o[32];
          tmem_ld32(tmem + ((uint32_t)(32 * warp) << 16) + kTaColO + 64 * j + 32 * half, o);
          tmem_wait_ld();
#pragma unroll
          for (int c = 0; c < 32; ++c) po[(size_t)(32 * half + c) * kTaDV + 128 * j + 32 * warp + lane] = __uint_as_float(o[c]);
        }
      }
      if (warp < kTaSoftmaxWarps && row_ok) {
        my_ml[head * 2] = m_ref * 0.6931471805599453f;  // back to natural units
        my_ml[head * 2 + 1] = l;
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0)
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"((uint32_t)kTaTmemCols) : "memory");
}

// Reads and clears the error word of the kernels above (0: no wait ever gave up).
int mla_attend_tc_take_error(unsigned *out) {
  unsigned zero = 0;
  BLOK_CUDA(cudaMemcpyFromSymbol(out, g_mla_tc_error, sizeof(unsigned)));
  if (*out) BLOK_CUDA(cudaMemcpyToSymbol(g_mla_tc_error, &zero, sizeof(unsigned)));
  return BLOK_OK;
}

// BLOK_MLA_TRACE=1 in the environment at the first launch: CTA (0, 0) of every launch records the time stamps described
// in the kernel; blok_mla_attend_trace copies them out.
static long long *g_trace_buf = nullptr;
static long long *trace_buffer() {
  static bool asked = false;
  if (!asked) {
    asked = true;
    const char *e = getenv("BLOK_MLA_TRACE");
    if (e && e[0] == '1' && cudaMalloc(&g_trace_buf, kTaTraceTiles * 16 * sizeof(long long)) == cudaSuccess)
      cudaMemset(g_trace_buf, 0, kTaTraceTiles * 16 * sizeof(long long));
  }
  return g_trace_buf;
}
int mla_attend_tc_trace(long long *host_out, int max_entries) {
  if (!g_trace_buf) return 0;
  const int n = max_entries < kTaTraceTiles * 16 ? max_entries : kTaTraceTiles * 16;
  if (cudaDeviceSynchronize() != cudaSuccess || cudaMemcpy(host_out, g_trace_buf, (size_t)n * sizeof(long long), cudaMemcpyDeviceToHost) != cudaSuccess)
    return 0;
  return n;
}

int launch_mla_attend_tc(const uint16_t *q, const uint16_t *cache, long ctx_stride, const int *seq_len, int B, int splits,
                         float scale, float *part_o, float *part_ml, cudaStream_t stream) {
  static bool configured = false;
  if (!configured) {
    BLOK_CUDA(cudaFuncSetAttribute(mla_attend_tc_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kTaSmemBytes));
    configured = true;
  }
  mla_attend_tc_kernel<false><<<dim3(splits, B), kTaThreads, kTaSmemBytes, stream>>>(q, cache, ctx_stride, seq_len, scale, part_o,
                                                                                     part_ml, nullptr, nullptr, 0, 0, trace_buffer());
  return launch_status("mla_attend_tc_kernel");
}

// The same over a paged pool: page_rows must be a positive multiple of the 64-token tile.
int launch_mla_attend_tc_paged(const uint16_t *q, const uint16_t *pool, const int *block_table, const int *slot_of,
                               int table_stride, int page_rows, const int *seq_len, int B, int splits, float scale, float *part_o,
                               float *part_ml, cudaStream_t stream) {
  static bool configured = false;
  if (!configured) {
    BLOK_CUDA(cudaFuncSetAttribute(mla_attend_tc_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kTaSmemBytes));
    configured = true;
  }
  mla_attend_tc_kernel<true><<<dim3(splits, B), kTaThreads, kTaSmemBytes, stream>>>(q, pool, 0, seq_len, scale, part_o, part_ml,
                                                                                    block_table, slot_of, table_stride, page_rows,
                                                                                    trace_buffer());
  return launch_status("mla_attend_tc_kernel(paged)");
}

}  // namespace blok
