// The attention core of absorbed MLA decode on the 5th-generation tensor cores (tcgen05, accumulators in tensor
// memory), its cache tiles brought in by TMA: one pass over the bf16 latent cache with an online softmax, split over
// the sequence (flash-decoding).  Replaces attn_tile_score_k / max / sum / accum (src/kimi_exec.cu:414-475) and the
// three-pass tiled_attention (:692-716).  Same interface and partial results as mla_attend_kernel (mla_attend.cu),
// which stays as the fallback.
//
// All 64 heads of a sequence share one latent row per token: per token 1,152 bytes are read once from HBM and feed
// 64 x (576 + 512) multiply-adds.  A CTA owns one (sequence, token range) and walks it in tiles of 64 tokens:
//
//   S [heads x tokens]     = Q [heads x 576] . C^T          36 MMAs M64 N64 K16: A = Q (shared memory, K-major, no
//                                                            swizzle), B = the tile read K-major; two partial sums
//   P = exp2(S * scale * log2 e - m)                         one head row per thread (tcgen05.ld), bf16, to shared memory
//   O^T [latent x heads]  += C^T [latent x tokens] . P^T     16 MMAs M128 N64 K16: A = the SAME tile bytes read MN-major
//                                                            (four blocks of 128 latent columns), B = P (K-major)
//
// A tile lies in shared memory as nine chunks of [64 tokens x 128 bytes] in the 128-byte swizzle, each written by one
// cp.async.bulk.tensor (no multicast; the tensor map covers this GPU's cache only).  Read K-major a chunk is 64 columns
// of a [64 tokens x 576] operand; read MN-major the same bytes are 64 rows of a [512 x 64 tokens] operand: one copy from
// HBM serves both products, and no thread touches the bytes on their way.
//
// The running maximum is kept lazily: a head's reference m changes only when a tile's maximum exceeds it by more than
// 40 (natural units); then all four consumer warps rescale O^T in tensor memory.  exp(s - m) stays far inside fp32 and
// bf16 range meanwhile, and the merge over the splits needs a consistent (m, sum, O) only.
//
// Warps: 0..3 consumers (the M = 64 accumulator S keeps head rows 16 w .. 16 w + 15 in lanes 0..15 of warp w's quarter of
// tensor memory; all four own the 128 lanes of O^T), 4: the TMA producer, 5: one lane issues the MMAs.  Every mbarrier
// wait is bounded; on a timeout the CTA records an error, still releases its tensor memory and returns.
#include <cuda.h>

#include <mutex>

#include "common.cuh"
#include "tmem_io.cuh"

namespace blok {

constexpr int kTaHeads = 64, kTaD = 576, kTaDV = 512;
constexpr int kTaTile = 64;                              // tokens per tile
constexpr int kTaChunks = kTaD / 64;                     // 128-byte column chunks of a cache row
constexpr int kTaChunkBytes = kTaTile * 128;             // 8,192
constexpr int kTaTileBytes = kTaChunks * kTaChunkBytes;  // 73,728
constexpr int kTaLbo = kTaHeads * 16;                    // Q and P (64 rows, no swizzle): bytes between 16-byte column groups
constexpr int kTaSbo = 128;                              // ... and between 8-row groups
constexpr int kTaQBytes = (kTaD / 8) * kTaLbo;           // 73,728
constexpr int kTaPBytes = (kTaTile / 8) * kTaLbo;        // P: [64 heads x 64 tokens] bf16, K (token) major
constexpr int kTaSmemBytes = 2 * kTaTileBytes + kTaQBytes + kTaPBytes + 1024;  // + 1024: the tiles start on a 1,024-byte boundary
constexpr int kTaConsumers = 128;
constexpr int kTaThreads = kTaConsumers + 64;
constexpr int kTaTmemCols = 512;                         // S: 2 buffers x 2 partial sums x 64 columns, O^T: 4 x 64 columns
constexpr int kTaColO = 256;
constexpr unsigned kTaSpinLimit = 1u << 21;
constexpr float kTaLazy = 57.7f;                         // 40 natural units in the log2 domain
constexpr int kTaTraceTiles = 64;

__device__ unsigned g_mla_tc_error = 0;

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
__device__ __forceinline__ void ta_cp16(uint32_t dst, const void *src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
// Shared-memory matrix descriptors (start address, leading and stride byte offsets in 16-byte units, version 1).
// No swizzle, K-major (Q and P): leading = between 16-byte column groups along K, stride = between 8-row groups.
__device__ __forceinline__ uint64_t ta_desc_plain(uint32_t saddr, uint32_t lbo, uint32_t sbo) {
  return (uint64_t)((saddr & 0x3FFFFu) >> 4) | ((uint64_t)(lbo >> 4) << 16) | ((uint64_t)(sbo >> 4) << 32) | (1ull << 46);
}
// 128-byte swizzle (layout type 2).  K-major: rows of 128 bytes, stride = 1,024 between 8-row groups, leading unused
// (1); a K = 16 step inside the 128-byte row advances the start address by 32 bytes.  MN-major: 64 contiguous
// elements along M, leading = between 64-element chunks along M, stride = 1,024 between 8-row groups along K.
__device__ __forceinline__ uint64_t ta_desc_sw128(uint32_t saddr, uint32_t lbo, uint32_t sbo) {
  return (uint64_t)((saddr & 0x3FFFFu) >> 4) | ((uint64_t)(lbo >> 4) << 16) | ((uint64_t)(sbo >> 4) << 32) | (1ull << 46) | (2ull << 61);
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
__device__ __forceinline__ void ta_expect_tx(uint32_t mbar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(mbar), "r"(bytes) : "memory");
}
// One box of the 2-D tensor map (x: column in elements, a multiple of 64; y: cache row) into shared memory; the bytes
// are counted on the mbarrier.
__device__ __forceinline__ void ta_tma_2d(uint32_t dst, const CUtensorMap *map, int x, int y, uint32_t mbar) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
               "l"(map), "r"(x), "r"(y), "r"(mbar)
               : "memory");
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

// grid = (splits, B); arguments as mla_attend_kernel, plus the tensor map of the cache ([rows, 576] bf16, boxes of
// 64 rows x 64 columns, 128-byte swizzle).  PAGED: page_rows is a multiple of the 64-token tile.
template <bool PAGED>
__global__ void __launch_bounds__(kTaThreads, 1)
    mla_attend_tc_kernel(const __grid_constant__ CUtensorMap tmap, const uint16_t *__restrict__ q, const uint16_t *__restrict__ cache,
                         long ctx_stride, const int *__restrict__ seq_len, float scale, float *__restrict__ part_o,
                         float *__restrict__ part_ml, const int *__restrict__ block_table, const int *__restrict__ slot_of,
                         int table_stride, int page_rows, long long *__restrict__ trace) {
  extern __shared__ unsigned char smem_raw[];
  __shared__ __align__(8) unsigned long long s_bar[11];
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
  // the swizzle is a function of the address: the tiles start on a 1,024-byte boundary
  const uint32_t raw = (uint32_t)__cvta_generic_to_shared(smem_raw);
  const uint32_t sT = (raw + 1023u) & ~1023u;
  unsigned char *smem = smem_raw + (sT - raw);
  const uint32_t sQ = sT + 2 * kTaTileBytes;
  const uint32_t sP = sQ + kTaQBytes;
  unsigned char *Pp = smem + 2 * kTaTileBytes + kTaQBytes;
  const uint32_t bar0 = (uint32_t)__cvta_generic_to_shared(&s_bar[0]);
  // tma[buf]: the tile's bytes have landed; fix[buf]: the rows past the sequence's end are zeroed (its last tile only);
  // sfull[buf]: the S MMAs' commit; sfree[buf]: the softmax warps have read S; pfull: they have written P;
  // empty[buf]: the commit behind the tile's P.C MMAs (tile buffer and P are free)
  const uint32_t bar_tma = bar0, bar_fix = bar0 + 16, bar_sfull = bar0 + 32, bar_sfree = bar0 + 48, bar_pfull = bar0 + 64,
                 bar_empty = bar0 + 72;
  if (tid == 0) {
    for (int i = 0; i < 2; ++i) {
      asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(bar_tma + 8 * i) : "memory");
      asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(bar_fix + 8 * i) : "memory");
      asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(bar_sfull + 8 * i) : "memory");
      asm volatile("mbarrier.init.shared::cta.b64 [%0], 4;" ::"r"(bar_sfree + 8 * i) : "memory");
      asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(bar_empty + 8 * i) : "memory");
    }
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 4;" ::"r"(bar_pfull) : "memory");
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"((uint32_t)__cvta_generic_to_shared(&s_tmem)),
                 "r"((uint32_t)kTaTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  {
    // Q [64 heads x 576] into 8 x 16-byte core matrices: consecutive threads take consecutive heads of one column group
    const uint16_t *qb = q + (size_t)b * kTaHeads * kTaD;
    for (int u = tid; u < kTaHeads * (kTaD / 8); u += kTaThreads) {
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
  // diagnostics (trace != NULL): CTA (0, 0) stamps, per tile, [0] buffer free, [1] TMA issued, [2] S issued, [3] S seen
  // by the softmax warps, [4] P handed over, [5] P.C issued, [8] S read, [9] softmax done (nanoseconds)
  auto stamp = [&](int n, int slot) {
    if (trace && blockIdx.x == 0 && blockIdx.y == 0 && n < kTaTraceTiles) {
      long long t;
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
      trace[n * 16 + slot] = t;
    }
  };
  // the sequence's last tile may hold rows past its end
  const int last_partial = (seq % kTaTile != 0 && te == ntiles) ? nt - 1 : -1;

  if (warp == 4) {
    // ---- the producer: nine boxes per tile, all counted on the buffer's mbarrier ----
    const uint16_t *cache_b = PAGED ? cache : cache + (size_t)b * ctx_stride * kTaD;
    const int *table_b = PAGED ? block_table + (size_t)(slot_of ? slot_of[b] : b) * table_stride : nullptr;
    auto first_row = [&](int tok0) -> long {  // the tensor map's row of the tile's first token
      if (PAGED) return (long)table_b[tok0 / page_rows] * page_rows + tok0 % page_rows;
      return (long)b * ctx_stride + tok0;
    };
    for (int n = 0; n < nt; ++n) {
      const int buf = n & 1;
      if (n >= 2 && !ta_wait(bar_empty + 8 * buf, (uint32_t)(((n >> 1) - 1) & 1), 1u)) {
        failed = true;
        break;
      }
      const int tok0 = (ts + n) * kTaTile;
      const uint32_t dst = sT + buf * kTaTileBytes;
      if (lane == 0) {
        stamp(n, 0);
        const int row = (int)first_row(tok0);
        ta_expect_tx(bar_tma + 8 * buf, kTaTileBytes);
#pragma unroll
        for (int c = 0; c < kTaChunks; ++c) ta_tma_2d(dst + c * kTaChunkBytes, &tmap, 64 * c, row, bar_tma + 8 * buf);
        if (n + 2 < nt) {
          // The buffer's next tile starts its way from HBM to L2 now: by the time the buffer is free again (this
          // tile's two products later) the copy finds it there, and HBM has been busy meanwhile.  A tile is contiguous
          // (dense cache, or inside a page); only rows of the sequence are touched.
          const int ptok = tok0 + 2 * kTaTile;
          const int prow = min(kTaTile, seq - ptok);
          const uint16_t *pp = PAGED ? cache + (size_t)first_row(ptok) * kTaD : cache_b + (size_t)ptok * kTaD;
          asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(pp), "r"((uint32_t)(prow * kTaD * 2)) : "memory");
        }
        stamp(n, 1);
      }
      if (n == last_partial) {
        // rows past the sequence's end hold whatever the allocation holds: zero them (their P is zero, and zero times
        // a stray NaN would not be), whole 128-byte rows, which the swizzle only permutes within
        if (!ta_wait(bar_tma + 8 * buf, (uint32_t)((n >> 1) & 1), 10u)) {
          failed = true;
          break;
        }
        const int valid = seq - tok0;
        unsigned char *tile = smem + (size_t)buf * kTaTileBytes;
        for (int idx = lane; idx < (kTaTile - valid) * kTaChunks * 8; idx += 32) {
          const int r = valid + idx / (kTaChunks * 8), rem = idx % (kTaChunks * 8);
          *reinterpret_cast<uint4 *>(tile + (rem >> 3) * kTaChunkBytes + r * 128 + (rem & 7) * 16) = make_uint4(0, 0, 0, 0);
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
        if (lane == 0) ta_arrive(bar_fix + 8 * buf);
      }
    }
  } else if (warp == 5) {
    if (lane == 0) {
      // ---- the MMA thread ----
      const uint32_t idesc_128 = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(kTaTile >> 3) << 17) | ((128u >> 4) << 24);
      const uint32_t idesc_s = (idesc_128 & ~(31u << 24)) | ((64u >> 4) << 24);  // M = 64
      const uint32_t idesc_pv = idesc_128 | (1u << 15);                          // A (the tile) MN-major
      const uint64_t q_desc = ta_desc_plain(sQ, kTaLbo, kTaSbo);
      const uint64_t p_desc = ta_desc_plain(sP, kTaLbo, kTaSbo);
      auto tile_ready = [&](int n, bool block) -> bool {  // the tile has landed (and, if it is the partial one, is zeroed)
        const int buf = n & 1;
        if (block) {
          if (!ta_wait(bar_tma + 8 * buf, (uint32_t)((n >> 1) & 1), 2u)) return false;
          if (n == last_partial && !ta_wait(bar_fix + 8 * buf, 0u, 4u)) return false;
          return true;
        }
        return ta_test(bar_tma + 8 * buf, (uint32_t)((n >> 1) & 1)) && (n != last_partial || ta_test(bar_fix + 8 * buf, 0u));
      };
      auto issue_s = [&](int n) {
        const int buf = n & 1;
        // every descriptor below is a per-tile base plus a constant: the start address sits in the low bits (16-byte units,
        // 14 bits for 256 KB) and no offset used here carries out of them
        const uint64_t c_desc = ta_desc_sw128(sT + buf * kTaTileBytes, 16, 1024);
#pragma unroll
        for (int c = 0; c < kTaChunks; ++c) {
#pragma unroll
          for (int k4 = 0; k4 < 4; ++k4) {
            const int kk = 4 * c + k4;  // K step of 16 columns: two column groups of Q, 32 bytes of the chunk's rows
            // even and odd K steps accumulate into two partial sums: an MMA of this size is shorter than the wait for the
            // previous one's accumulator, and two chains halve that wait
            ta_mma(tmem + 128 * buf + 64 * (kk & 1), q_desc + (uint64_t)(kk * ((2 * kTaLbo) >> 4)),
                   c_desc + (uint64_t)((c * kTaChunkBytes + k4 * 32) >> 4), idesc_s, kk > 1 ? 1u : 0u);
          }
        }
        ta_commit(bar_sfull + 8 * buf);
        stamp(n, 2);
      };
      auto issue_pv = [&](int n) {
        const int buf = n & 1;
        const uint64_t a_desc = ta_desc_sw128(sT + buf * kTaTileBytes, kTaChunkBytes, 1024);
        // block j: latent columns [128 j, +128) = chunks 2 j and 2 j + 1; a K step is 16 tokens = two 8-row groups.  The
        // four blocks take turns: consecutive MMAs then accumulate into different columns of tensor memory and do not
        // wait for one another.
#pragma unroll
        for (int kk = 0; kk < kTaTile / 16; ++kk) {
#pragma unroll
          for (int j = 0; j < kTaDV / 128; ++j)
            ta_mma(tmem + kTaColO + 64 * j, a_desc + (uint64_t)((2 * j * kTaChunkBytes + kk * 2048) >> 4),
                   p_desc + (uint64_t)(kk * ((2 * kTaLbo) >> 4)), idesc_pv, (n > 0 || kk > 0) ? 1u : 0u);
        }
        ta_commit(bar_empty + 8 * buf);
        stamp(n, 5);
      };
      if (!tile_ready(0, true)) failed = true;
      if (!failed) {
        tc_fence_after();
        issue_s(0);
      }
      for (int n = 0; n < nt && !failed; ++n) {
        // the next tile's scores go first when that tile has landed already: they run under this tile's softmax
        bool early = false;
        const int nn = n + 1, nb = nn & 1;
        if (nn < nt && tile_ready(nn, false) && (nn < 2 || ta_test(bar_sfree + 8 * nb, (uint32_t)(((nn >> 1) - 1) & 1)))) {
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
          if (!tile_ready(nn, true) || (nn >= 2 && !ta_wait(bar_sfree + 8 * nb, (uint32_t)(((nn >> 1) - 1) & 1), 5u))) {
            failed = true;
            break;
          }
          tc_fence_after();
          issue_s(nn);
        }
      }
    }
  } else {
    // ---- consumers: lanes 0..15 of warp w hold head rows 16 w .. 16 w + 15 of S ----
    const float sl2 = scale * 1.4426950408889634f;
    float m_ref = -INFINITY, l = 0.f;
    const bool row_ok = lane < 16;
    const int head = 16 * warp + lane;
    for (int n = 0; n < nt; ++n) {
      const int buf = n & 1;
      uint32_t pk[kTaTile / 2];
      bool need = false;
      if (!failed && !ta_wait(bar_sfull + 8 * buf, (uint32_t)((n >> 1) & 1), 6u)) failed = true;
      if (!failed) {
        if (tid == 0) stamp(n, 3);
        tc_fence_after();
        uint32_t r[kTaTile];
        {
          uint32_t r2[kTaTile];  // the two partial sums of the score product
          tmem_ld64(tmem + ((uint32_t)(32 * warp) << 16) + 128 * buf, r);
          tmem_ld64(tmem + ((uint32_t)(32 * warp) << 16) + 128 * buf + 64, r2);
          tmem_wait_ld();
#pragma unroll
          for (int j = 0; j < kTaTile; ++j) r[j] = __float_as_uint(__uint_as_float(r[j]) + __uint_as_float(r2[j]));
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) ta_arrive(bar_sfree + 8 * buf);
        if (tid == 0) stamp(n, 8);
        const int tok0 = (ts + n) * kTaTile;
        if (tok0 + kTaTile > seq) {  // the sequence's last tile: tokens past the end take no weight
#pragma unroll
          for (int j = 0; j < kTaTile; ++j)
            if (tok0 + j >= seq) r[j] = 0xff800000u;
        }
        float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
#pragma unroll
        for (int j = 0; j < kTaTile; j += 4) {
          mx0 = fmaxf(mx0, __uint_as_float(r[j]));
          mx1 = fmaxf(mx1, __uint_as_float(r[j + 1]));
          mx2 = fmaxf(mx2, __uint_as_float(r[j + 2]));
          mx3 = fmaxf(mx3, __uint_as_float(r[j + 3]));
        }
        const float mx = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3)) * sl2;  // the scale is positive
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
        float sum0 = 0.f, sum1 = 0.f, sum2 = 0.f, sum3 = 0.f;
#pragma unroll
        for (int j = 0; j < kTaTile; j += 4) {
          // the probabilities enter the second product rounded to bf16 (as the reference rounds them, :466); the
          // normaliser sums the same rounded values
          const uint32_t pa = ta_pack_bf16x2(ta_ex2(fmaf(__uint_as_float(r[j]), sl2, nm)), ta_ex2(fmaf(__uint_as_float(r[j + 1]), sl2, nm)));
          const uint32_t pb = ta_pack_bf16x2(ta_ex2(fmaf(__uint_as_float(r[j + 2]), sl2, nm)), ta_ex2(fmaf(__uint_as_float(r[j + 3]), sl2, nm)));
          sum0 += __uint_as_float(pa << 16);
          sum1 += __uint_as_float(pa & 0xffff0000u);
          sum2 += __uint_as_float(pb << 16);
          sum3 += __uint_as_float(pb & 0xffff0000u);
          pk[j >> 1] = pa;
          pk[(j >> 1) + 1] = pb;
        }
        l = l * alpha + ((sum0 + sum1) + (sum2 + sum3));
        if (tid == 0) stamp(n, 9);
      }
      need = __any_sync(0xffffffffu, need);
      if (lane == 0) s_need[buf][warp] = need ? 1 : 0;
      if (ta_consumers_sync(failed)) {
        failed = true;
        break;
      }
      if (s_need[buf][0] | s_need[buf][1] | s_need[buf][2] | s_need[buf][3]) {
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
      if (!failed) {
        if (n > 0 && !ta_wait(bar_empty + 8 * ((n - 1) & 1), (uint32_t)(((n - 1) >> 1) & 1), 8u)) {
          failed = true;  // reaches the others at the next tile's barrier
        } else {
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
      if (row_ok) {
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
  if (cudaDeviceSynchronize() != cudaSuccess ||
      cudaMemcpy(host_out, g_trace_buf, (size_t)n * sizeof(long long), cudaMemcpyDeviceToHost) != cudaSuccess)
    return 0;
  return n;
}

// The tensor map of a cache of `rows` rows of 576 bf16 at `base`: boxes of 64 rows x 64 columns in the 128-byte swizzle;
// rows at or past `rows` read as zeros.  cuTensorMapEncodeTiled is resolved from the driver at run time; the last few
// maps are kept (a model's layers pass the same caches step after step).
typedef CUresult (*ta_encode_fn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                 const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                 CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static int cache_tensor_map(const uint16_t *base, long rows, CUtensorMap *out) {
  struct Entry {
    const void *base;
    long rows;
    CUtensorMap map;
  };
  static std::mutex mu;
  static Entry kept[128];
  static int n_kept = 0, next = 0;
  static ta_encode_fn encode = nullptr;
  std::lock_guard<std::mutex> lock(mu);
  for (int i = 0; i < n_kept; ++i)
    if (kept[i].base == base && kept[i].rows == rows) {
      *out = kept[i].map;
      return BLOK_OK;
    }
  if (!encode) {
    void *fn = nullptr;
    cudaDriverEntryPointQueryResult qres;
    BLOK_CUDA(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres));
    BLOK_REQUIRE(fn && qres == cudaDriverEntryPointSuccess, BLOK_ERR_CUDA, "blok_mla_decode: the driver has no cuTensorMapEncodeTiled");
    encode = reinterpret_cast<ta_encode_fn>(fn);
  }
  const cuuint64_t dims[2] = {(cuuint64_t)kTaD, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)kTaD * 2};
  const cuuint32_t box[2] = {64, (cuuint32_t)kTaTile};
  const cuuint32_t estr[2] = {1, 1};
  CUtensorMap map;
  const CUresult r = encode(&map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<uint16_t *>(base), dims, strides, box, estr,
                            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  BLOK_REQUIRE(r == CUDA_SUCCESS, BLOK_ERR_CUDA, "blok_mla_decode: cuTensorMapEncodeTiled failed (%d) for a cache of %ld rows at %p", (int)r,
               rows, (const void *)base);
  kept[next] = Entry{base, rows, map};
  next = (next + 1) % 128;
  if (n_kept < 128) ++n_kept;
  *out = map;
  return BLOK_OK;
}

// total_rows: the rows of the cache allocation from `cache` on (reads past them give zeros).
int launch_mla_attend_tc(const uint16_t *q, const uint16_t *cache, long ctx_stride, long total_rows, const int *seq_len, int B, int splits,
                         float scale, float *part_o, float *part_ml, cudaStream_t stream) {
  static bool configured = false;
  if (!configured) {
    BLOK_CUDA(cudaFuncSetAttribute(mla_attend_tc_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kTaSmemBytes));
    configured = true;
  }
  CUtensorMap map;
  if (int rc = cache_tensor_map(cache, total_rows, &map)) return rc;
  mla_attend_tc_kernel<false><<<dim3(splits, B), kTaThreads, kTaSmemBytes, stream>>>(map, q, cache, ctx_stride, seq_len, scale, part_o,
                                                                                     part_ml, nullptr, nullptr, 0, 0, trace_buffer());
  return launch_status("mla_attend_tc_kernel");
}

// The same over a paged pool of pool_rows rows: page_rows must be a positive multiple of the 64-token tile.
int launch_mla_attend_tc_paged(const uint16_t *q, const uint16_t *pool, long pool_rows, const int *block_table, const int *slot_of,
                               int table_stride, int page_rows, const int *seq_len, int B, int splits, float scale, float *part_o,
                               float *part_ml, cudaStream_t stream) {
  static bool configured = false;
  if (!configured) {
    BLOK_CUDA(cudaFuncSetAttribute(mla_attend_tc_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kTaSmemBytes));
    configured = true;
  }
  CUtensorMap map;
  if (int rc = cache_tensor_map(pool, pool_rows, &map)) return rc;
  mla_attend_tc_kernel<true><<<dim3(splits, B), kTaThreads, kTaSmemBytes, stream>>>(map, q, pool, 0, seq_len, scale, part_o, part_ml,
                                                                                    block_table, slot_of, table_stride, page_rows,
                                                                                    trace_buffer());
  return launch_status("mla_attend_tc_kernel(paged)");
}

}  // namespace blok
