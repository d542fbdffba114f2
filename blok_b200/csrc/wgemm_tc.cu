// Weight-streaming grouped GEMM on the 5th-generation tensor cores (tcgen05, accumulators
// in tensor memory) for the INT4 experts of the batched routed-MoE layer:
//   out[token, row] = sum_c bf16(q[row, c] * scale[row, c / 32]) * x[token, c]
// Reference arithmetic: matvec_i4_bf16_scale_k (src/kimi_exec.cu:300-323) applied per
// token; the dequantised weight is the reference's bf16(q * s) bit for bit (:312).
//
// One CTA = one tile of up to 64 tokens of one expert x two 128-row blocks of weights (gate
// and up rows of the same indices, or rows r and r + 128 of the down projection).  The
// weight rows are the M = 128 dimension of tcgen05.mma, the tokens the N dimension, so
// a weight byte is read from HBM and dequantised once per tile whatever the token
// count.  Eight producer warps (one weight row per thread) copy 256 packed columns and
// their scales per step into shared memory with coalesced cp.async (rows XOR-swizzled
// against bank conflicts), dequantise them exactly and write them to TENSOR MEMORY with
// tcgen05.st as the A operand, 64 columns per pipeline stage; the tile's activations go
// to shared memory in the K-major core-matrix layout the instruction reads (no swizzle:
// 8 rows x 16 bytes per core matrix) as the B operand.  A ninth warp's first lane issues
// the MMAs; producers arrive on a `full` mbarrier per stage, tcgen05.commit on an `empty`
// mbarrier frees it.  Every mbarrier wait is bounded; on a timeout the CTA records an
// error, still releases its tensor memory and returns.
#include <algorithm>

#include "common.cuh"
#include "wgemm.h"

namespace blok {

constexpr int kTcProducers = 256;    // threads that unpack weights: one weight row each
constexpr int kTcThreads = kTcProducers + 32;  // plus one warp whose first lane issues the MMAs
constexpr int kTcN = kWgTileTokens;  // token columns of a tile
constexpr int kTcKC = 64;            // weight columns per pipeline step
constexpr int kTcStages = 2;
constexpr int kTcSbo = 128;          // bytes between 8-token groups of the activation tile
constexpr int kTcBLbo = 1040;        // 8 token groups x 128 B, plus 16 B so that the 8 K-slices of a token hit 8 banks
constexpr int kTcBBytes = (kTcKC / 8) * kTcBLbo;
constexpr int kTcStageBytes = ((kTcBBytes + 127) / 128) * 128;  // shared memory per stage: the activation tile only
constexpr int kTcSuper = 256;        // weight columns per copy step: 128 packed bytes and 8 scales of each row
constexpr int kTcRing = 2;           // copy steps resident per CTA: one being unpacked, one in flight
constexpr int kTcRawBytes = kTcProducers * 128 + kTcProducers * 16;  // 256 rows x (128 B of words + 16 B of scales)
constexpr int kTcACols = kTcKC / 2;                       // tensor-memory columns of one 128-row block of one step (2 bf16 per column)
constexpr int kTcTmemCols = 256;                          // 2 accumulators x 64 columns + 2 stages x 2 blocks x 32 columns of weights
constexpr unsigned kTcSpinLimit = 1u << 22;

__device__ unsigned g_wgemm_tc_error = 0;

__device__ __forceinline__ uint32_t tc_bf16x2_sub(uint32_t a, uint32_t b) {
  uint32_t r;
  asm("sub.rn.bf16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
  return r;
}
__device__ __forceinline__ uint32_t tc_bf16x2_mul(uint32_t a, uint32_t b) {
  uint32_t r;
  asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
  return r;
}

// Exact dequantised pairs of one packed word: (bf16(q_j * s), bf16(q_{j+4} * s)), j = 0..3,
// i.e. the word's eight columns in the order 0 4 1 5 2 6 3 7 (the activations get the same order).
__device__ __forceinline__ uint4 tc_dequant_word(uint32_t w, uint32_t s2) {
  constexpr uint32_t kMask = 0x000f000fu, kMagic = 0x43004300u, kOff = 0x43084308u;  // 128.0 | nibble, 136.0
  uint32_t o[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    uint32_t v;
    asm("lop3.b32 %0, %1, %2, %3, 0xea;" : "=r"(v) : "r"(w >> (4 * j)), "r"(kMask), "r"(kMagic));
    o[j] = tc_bf16x2_mul(tc_bf16x2_sub(v, kOff), s2);
  }
  return make_uint4(o[0], o[1], o[2], o[3]);
}

// Shared-memory matrix descriptor, K-major, no swizzle: start address, leading (K) and
// stride (M/N) byte offsets in 16-byte units, descriptor version 1.
__device__ __forceinline__ uint64_t tc_smem_desc(uint32_t saddr, uint32_t lbo, uint32_t sbo) {
  return (uint64_t)((saddr & 0x3FFFFu) >> 4) | ((uint64_t)(lbo >> 4) << 16) | ((uint64_t)(sbo >> 4) << 32) | (1ull << 46);
}

__device__ __forceinline__ void tc_mma_f16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
      "}\n" ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// The same with the A operand (128 rows x 16 columns of bf16) taken from tensor memory.
__device__ __forceinline__ void tc_mma_f16_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t"
      "}\n" ::"r"(tmem_d), "r"(tmem_a), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}

__device__ __forceinline__ void tc_st32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, "
      "%19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]),
      "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]),
      "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]),
      "r"(r[31])
      : "memory");
}

__device__ __forceinline__ void tc_commit(uint32_t mbar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(mbar) : "memory");
}

// Bounded wait for the given phase parity of an mbarrier; false on timeout.
__device__ __forceinline__ bool tc_mbar_wait(uint32_t mbar, uint32_t parity) {
  for (unsigned it = 0; it < kTcSpinLimit; ++it) {
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
    __nanosleep(64);  // a failed try already waited out the hardware's own time slice; do not burn issue slots
  }
  return false;
}

__device__ __forceinline__ void tc_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}

__device__ __forceinline__ void tc_cp_async16(uint32_t dst, const void *src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void tc_cp_async4(uint32_t dst, const void *src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst), "l"(src) : "memory");
}

// Epilogue of a tile: lane l of warp w (8 warps) holds accumulator row 32 (w % 4) + l of both row blocks (its
// tensor-memory lane); warps 0..3 take the even 16-token column blocks, warps 4..7 the odd ones.
template <bool SWIGLU>
__device__ __forceinline__ void tc_epilogue(const WgArgs &a, uint32_t tmem, int acc1_col, int warp, int lane, int N, int cnt, int p0,
                                            int row0) {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const int lg = warp & 3, row = 32 * lg + lane;
  const uint32_t trow = tmem + ((uint32_t)(32 * lg) << 16);
  for (int n0 = 16 * (warp >> 2); n0 < N; n0 += 32) {
    uint32_t ra[16], rb[16];
    tc_ld16(trow + n0, ra);
    tc_ld16(trow + acc1_col + n0, rb);
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      const int tok = n0 + j;
      if (tok < cnt) {
        const size_t p = a.out_index ? (size_t)a.out_index[p0 + tok] : (size_t)(p0 + tok);
        const float va = __uint_as_float(ra[j]), vb = __uint_as_float(rb[j]);
        if (SWIGLU) {
          const float gv = round_bf16(va), uv = round_bf16(vb);
          const float m = round_bf16(round_bf16(gv / (1.0f + expf(-gv))) * uv);
          a.out_bf16[p * a.R + row0 + row] = f32_to_bf16_bits(m);
        } else if (a.out_f32) {
          a.out_f32[p * a.R + row0 + row] = va;
          a.out_f32[p * a.R + row0 + 128 + row] = vb;
        } else {
          a.out_bf16[p * a.R + row0 + row] = f32_to_bf16_bits(va);
          a.out_bf16[p * a.R + row0 + 128 + row] = f32_to_bf16_bits(vb);
        }
      }
    }
  }
}

template <bool SWIGLU>
__global__ void __launch_bounds__(kTcThreads, 2) wgemm_tc_kernel(const WgArgs a) {
  extern __shared__ __align__(128) unsigned char smem[];
  __shared__ __align__(8) unsigned long long s_mbar[2 * kTcStages];
  __shared__ uint32_t s_tmem_base;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  // The grid's y extent is a fixed number of tile slots, not the worst-case tile count (tokens / 64 + experts, most of
  // which a launch does not use or leaves to the small-group kernel: 6,000-11,000 CTAs that only start and leave cost
  // 36-58 us per launch); a CTA walks the tiles slot, slot + slots, ...
  const int ntiles = *a.num_tiles;
  const int skip_upto = a.small_max ? (a.small_limit ? *a.small_limit : a.small_max) : 0;  // groups wgemv_small.cu has taken
  bool have_tmem = false;
  uint32_t tmem = 0;
  for (int tile = blockIdx.y; tile < ntiles; tile += gridDim.y) {
  const int e = a.tile_expert[tile], p0 = a.tile_start[tile], cnt = a.tile_count[tile];
  if (cnt <= skip_upto) continue;  // nothing is allocated yet
  const int N = max(16, (cnt + 15) & ~15);  // token columns the MMAs cover

  // ---- this thread unpacks weight row r of block blk: threads 0..127 block 0 (gate rows / rows r), 128..255 block 1 ----
  const int blk = tid >> 7, r = tid & 127;
  const int rows_per_cta = SWIGLU ? 128 : 256;
  const int row0 = blockIdx.x * rows_per_cta;
  const size_t rowbytes = (size_t)a.K / 2;  // packed bytes per weight row
  const size_t srowbytes = (size_t)a.K / 16;  // scale bytes per weight row
  const size_t grow0 = (size_t)e * a.expert_stride_rows + row0;
  const unsigned char *wbase0 = reinterpret_cast<const unsigned char *>(a.w_a) + grow0 * rowbytes;
  const unsigned char *wbase1 = SWIGLU ? reinterpret_cast<const unsigned char *>(a.w_b) + grow0 * rowbytes : wbase0 + 128 * rowbytes;
  const unsigned char *sbase0 = reinterpret_cast<const unsigned char *>(a.s_a) + grow0 * srowbytes;
  const unsigned char *sbase1 = SWIGLU ? reinterpret_cast<const unsigned char *>(a.s_b) + grow0 * srowbytes : sbase0 + 128 * srowbytes;
  // ---- this thread's two pieces of the activation tile: token (tid / 8) + 32 i, K-slice tid % 8 ----
  const int ki = tid & 7;
  const uint4 *xp[2];
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int tok = (tid >> 3) + 32 * i;
    xp[i] = nullptr;
    if (tok < cnt) {
      const size_t xr = a.x_index ? (size_t)a.x_index[p0 + tok] : (size_t)(p0 + tok);
      xp[i] = reinterpret_cast<const uint4 *>(a.x + xr * a.K) + ki;
    }
  }
  // Packed words and scales reach shared memory in copy steps of 256 columns: 8 neighbouring lanes copy the 128
  // contiguous bytes of one row (16 bytes each), so a warp's cp.async touches 4 cache lines, not 32.  Piece p of row
  // q lands at q * 128 + ((p ^ (q & 7)) * 16): both the copy and the later per-row reads are free of bank conflicts.
  // The activations (L2 resident, shared by all row blocks of the expert) are fetched one step ahead into registers.
  const uint32_t sbase = (uint32_t)__cvta_generic_to_shared(smem);
  const uint32_t raw0 = sbase + kTcStages * kTcStageBytes;
  const unsigned char *rawp = smem + kTcStages * kTcStageBytes;
  const int nchunks = a.K / kTcKC;
  const int nsuper = a.K / kTcSuper;
  const bool producer = tid < kTcProducers;
  auto issue = [&](int sc) {
    if (sc < nsuper) {
      const uint32_t slot = raw0 + (uint32_t)(sc % kTcRing) * kTcRawBytes;
      const int q0 = tid >> 3, pc = tid & 7;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int q = q0 + 32 * i;  // 0..255: block q / 128, row q % 128
        const unsigned char *src = (i < 4 ? wbase0 : wbase1) + (size_t)(q & 127) * rowbytes + (size_t)sc * 128 + pc * 16;
        tc_cp_async16(slot + q * 128 + ((pc ^ (q & 7)) * 16), src);
      }
      tc_cp_async16(slot + kTcProducers * 128 + tid * 16, (blk ? sbase1 : sbase0) + (size_t)r * srowbytes + (size_t)sc * 16);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  auto fetch_x = [&](int c, uint4 (&xv)[2]) {
#pragma unroll
    for (int i = 0; i < 2; ++i) xv[i] = xp[i] ? __ldg(xp[i] + (size_t)c * (kTcKC / 8)) : make_uint4(0, 0, 0, 0);
  };
  if (producer) issue(0);

  // ---- barriers and tensor memory: full[s] counts the 8 producer warps, empty[s] the MMAs' commit ----
  const uint32_t mbar_full = (uint32_t)__cvta_generic_to_shared(&s_mbar[0]);
  const uint32_t mbar_empty = mbar_full + 8 * kTcStages;
  if (tid == 0) {
#pragma unroll
    for (int s = 0; s < kTcStages; ++s) {
      asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(mbar_full + 8 * s), "r"(kTcProducers / 32) : "memory");
      asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(mbar_empty + 8 * s) : "memory");
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 0 && !have_tmem) {  // once per CTA, at its first tile; the columns serve every tile the CTA walks
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"((uint32_t)__cvta_generic_to_shared(&s_tmem_base)),
                 "r"((uint32_t)kTcTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  have_tmem = true;
  uint4 xnext[2];
  if (producer) fetch_x(0, xnext);
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  tmem = s_tmem_base;
  const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(N >> 3) << 17) | ((128u >> 4) << 24);

  bool failed = false;
  if (producer) {
    // ---- producers: unpack step c into stage c % 2 as soon as the MMAs of step c - 2 have released it ----
    for (int sc = 0; sc < nsuper; ++sc) {
      asm volatile("cp.async.wait_group 0;" ::: "memory");  // this thread's copies of the step have landed
      // producers' barrier: everybody's copies have landed and the other slot is no longer read.  It also ORs the
      // threads' failure flags, so that after a timeout all of them leave together and nobody waits here alone.
      uint32_t anyfail;
      asm volatile(
          "{\n\t"
          ".reg .pred p, q;\n\t"
          "setp.ne.u32 q, %1, 0;\n\t"
          "bar.red.or.pred p, 1, %2, q;\n\t"
          "selp.u32 %0, 1, 0, p;\n\t"
          "}\n"
          : "=r"(anyfail)
          : "r"((uint32_t)failed), "n"(kTcProducers)
          : "memory");
      if (anyfail) {
        failed = true;
        break;
      }
      issue(sc + 1);
      const unsigned char *raw = rawp + (size_t)(sc % kTcRing) * kTcRawBytes;
      const uint4 scq = *reinterpret_cast<const uint4 *>(raw + kTcProducers * 128 + tid * 16);  // the row's 8 scales
      const uint32_t scw[4] = {scq.x, scq.y, scq.z, scq.w};
#pragma unroll
      for (int j = 0; j < kTcSuper / kTcKC; ++j) {
        const int c = sc * (kTcSuper / kTcKC) + j;
        uint4 xcur[2];
#pragma unroll
        for (int i = 0; i < 2; ++i) xcur[i] = xnext[i];
        if (c + 1 < nchunks) fetch_x(c + 1, xnext);
        const int s = c % kTcStages;
        if (c >= kTcStages && !tc_mbar_wait(mbar_empty + 8 * s, (uint32_t)((c / kTcStages - 1) & 1))) {
          failed = true;
          break;
        }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        unsigned char *B = smem + (size_t)s * kTcStageBytes;
        // The row's 64 dequantised weights of this step go to tensor memory as the MMA's A operand: lane = row, two
        // bf16 per 32-bit column, 8 columns per K = 16 step (column pairs in the order 0 4 1 5 2 6 3 7 of each word).
        uint32_t av[32];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const uint32_t s2 = __byte_perm(scw[j], scw[j], h ? 0x3232 : 0x1010);
          const uint4 q = *reinterpret_cast<const uint4 *>(raw + tid * 128 + (((2 * j + h) ^ (tid & 7)) * 16));
          const uint32_t qw[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
          for (int w = 0; w < 4; ++w) {
            const uint4 d = tc_dequant_word(qw[w], s2);
            av[(h * 4 + w) * 4 + 0] = d.x;
            av[(h * 4 + w) * 4 + 1] = d.y;
            av[(h * 4 + w) * 4 + 2] = d.z;
            av[(h * 4 + w) * 4 + 3] = d.w;
          }
        }
        tc_st32(tmem + ((uint32_t)(32 * (warp & 3)) << 16) + 2 * kTcN + (uint32_t)(s * 2 + blk) * kTcACols, av);
#pragma unroll
        for (int i = 0; i < 2; ++i) {
          if (32 * i < N) {
            const uint4 v = xcur[i];
            uint4 o;  // columns 0 4 1 5 2 6 3 7, as the weights
            o.x = __byte_perm(v.x, v.z, 0x5410);
            o.y = __byte_perm(v.x, v.z, 0x7632);
            o.z = __byte_perm(v.y, v.w, 0x5410);
            o.w = __byte_perm(v.y, v.w, 0x7632);
            const int tok = (tid >> 3) + 32 * i;
            *reinterpret_cast<uint4 *>(B + ki * kTcBLbo + (tok >> 3) * kTcSbo + (tok & 7) * 16) = o;
          }
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // the activation tile is read by the tensor core's proxy
        asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncwarp();
        if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(mbar_full + 8 * s) : "memory");
      }
    }
    // all MMAs have completed once the last step's commit has arrived
    if (!failed) {
      const int last = nchunks - 1;
      failed = !tc_mbar_wait(mbar_empty + 8 * (last % kTcStages), (uint32_t)((last / kTcStages) & 1));
    }
  } else if (lane == 0) {
    // ---- the MMA thread: 4 K = 16 steps x 2 row blocks per stage, then the commit that releases the stage ----
    for (int c = 0; c < nchunks; ++c) {
      const int s = c % kTcStages;
      if (!tc_mbar_wait(mbar_full + 8 * s, (uint32_t)((c / kTcStages) & 1))) {
        failed = true;
        break;
      }
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint32_t b = sbase + (uint32_t)s * kTcStageBytes;
      const uint32_t ta = tmem + 2 * kTcN + (uint32_t)(s * 2) * kTcACols;
#pragma unroll
      for (int j = 0; j < kTcKC / 16; ++j) {
        const uint32_t acc = (c > 0 || j > 0) ? 1u : 0u;
        const uint64_t bd = tc_smem_desc(b + j * 2 * kTcBLbo, kTcBLbo, kTcSbo);
        tc_mma_f16_ts(tmem, ta + 8 * j, bd, idesc, acc);
        tc_mma_f16_ts(tmem + kTcN, ta + kTcACols + 8 * j, bd, idesc, acc);
      }
      tc_commit(mbar_empty + 8 * s);
    }
  }
  failed = __any_sync(0xffffffffu, failed);  // warp-uniform: the tensor-memory loads below are warp-wide
  if (failed && lane == 0) atomicExch(&g_wgemm_tc_error, 1u);

  if (producer && !failed) tc_epilogue<SWIGLU>(a, tmem, kTcN, warp, lane, N, cnt, p0, row0);
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  // a CTA that gave up on a barrier stops here (every warp: the flag goes through the barrier's OR)
  if (__syncthreads_or(failed ? 1 : 0)) break;
  // the next tile sets the barriers up afresh
  if (tid == 0) {
#pragma unroll
    for (int s = 0; s < 2 * kTcStages; ++s) asm volatile("mbarrier.inval.shared::cta.b64 [%0];" ::"r"(mbar_full + 8 * s) : "memory");
  }
  __syncthreads();
  }
  if (have_tmem && warp == 0)  // block-uniform: every thread walked the same tiles
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"((uint32_t)kTcTmemCols) : "memory");
}

// ---- bf16 weights (shared expert): both operands come straight from global memory into the core-matrix layout
// with 16-byte cp.async copies, one per (row, 8-column slice); no registers, no permutation.  kBfStages steps of
// 2 x 128 weight rows + the token tile are in flight per CTA. ----
constexpr int kBfMinSteps = 4;       // fewest 64-column steps the pipelines below are written for
constexpr int kBfALbo = 2048 + 16;   // + 16 B: the 8 K-slices of a row, copied by 8 neighbouring lanes, hit 8 banks
constexpr int kBfABytes = (kTcKC / 8) * kBfALbo;
// NT = token columns per tile: 64 for tiles of an expert group, 256 for a dense layer (every token, same weights),
// where the larger tile halves the bytes fetched from L2 per flop.  STAGES steps are resident per CTA.
template <int NT>
struct BfCfg {
  static constexpr int kBLbo = (NT / 8) * 128 + 16;
  static constexpr int kBBytes = (kTcKC / 8) * kBLbo;
  static constexpr int kStageBytes = ((2 * kBfABytes + kBBytes + 127) / 128) * 128;
  static constexpr int kStages = NT == 64 ? 4 : 3;
  static constexpr int kTmemCols = 2 * NT;
};

__device__ __forceinline__ void tc_cp_async16_zfill(uint32_t dst, const void *src, uint32_t src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}

template <bool SWIGLU, int NT>
__global__ void __launch_bounds__(kTcThreads, 1) wgemm_tc_bf16_kernel(const WgArgs a) {
  using Cfg = BfCfg<NT>;
  constexpr int kBfStages = Cfg::kStages;
  constexpr int kBfStageBytes = Cfg::kStageBytes;
  constexpr int kBfTmemCols = Cfg::kTmemCols;
  constexpr int kBLbo = Cfg::kBLbo;
  extern __shared__ __align__(128) unsigned char smem[];
  __shared__ __align__(8) unsigned long long s_mbar[2 * kBfStages];
  __shared__ uint32_t s_tmem_base;
  const int tile = blockIdx.y;
  int e, p0, cnt;
  if (a.identity_tiles) {  // dense: tile t covers rows [NT t, NT t + NT) of x
    e = 0;
    p0 = NT * tile;
    cnt = min(NT, a.n_rows - p0);
    if (cnt <= 0) return;
  } else {
    if (tile >= *a.num_tiles) return;
    e = a.tile_expert[tile], p0 = a.tile_start[tile], cnt = a.tile_count[tile];
  }
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int N = max(16, (cnt + 15) & ~15);
  const int rows_per_cta = SWIGLU ? 128 : 256;
  const int row0 = blockIdx.x * rows_per_cta;
  const bool producer = tid < kTcProducers;
  const int nchunks = a.K / kTcKC;
  const uint32_t sbase = (uint32_t)__cvta_generic_to_shared(smem);

  // this thread's pieces: weight rows (tid / 8) + 32 i of both blocks (i < 4), tokens (tid / 8) + 32 i (i < 2), K-slice tid % 8
  const int ki = tid & 7, r0 = tid >> 3;
  const size_t rowbytes = (size_t)a.K * 2;
  const unsigned char *wa = reinterpret_cast<const unsigned char *>(a.w_a) + ((size_t)e * a.expert_stride_rows + row0 + r0) * rowbytes + ki * 16;
  const unsigned char *wb = SWIGLU ? reinterpret_cast<const unsigned char *>(a.w_b) + ((size_t)e * a.expert_stride_rows + row0 + r0) * rowbytes + ki * 16
                                   : wa + 128 * rowbytes;
  constexpr int kXPieces = NT / 32;  // activation pieces per thread and step
  const unsigned char *xs[kXPieces];
  uint32_t xbytes[kXPieces];
#pragma unroll
  for (int i = 0; i < kXPieces; ++i) {
    const int tok = r0 + 32 * i;
    xs[i] = reinterpret_cast<const unsigned char *>(a.x);
    xbytes[i] = 0;  // rows beyond the tile's tokens are filled with zeros
    if (tok < cnt) {
      const size_t xr = a.x_index ? (size_t)a.x_index[p0 + tok] : (size_t)(p0 + tok);
      xs[i] = reinterpret_cast<const unsigned char *>(a.x) + xr * rowbytes + ki * 16;
      xbytes[i] = 16;
    }
  }
  auto issue = [&](int c) {
    if (c < nchunks) {
      const uint32_t st = sbase + (uint32_t)(c % kBfStages) * kBfStageBytes;
      const size_t koff = (size_t)c * (kTcKC * 2);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int row = r0 + 32 * i;
        const uint32_t d = (uint32_t)(ki * kBfALbo + (row >> 3) * kTcSbo + (row & 7) * 16);
        tc_cp_async16(st + d, wa + (size_t)(32 * i) * rowbytes + koff);
        tc_cp_async16(st + kBfABytes + d, wb + (size_t)(32 * i) * rowbytes + koff);
      }
#pragma unroll
      for (int i = 0; i < kXPieces; ++i) {
        const int tok = r0 + 32 * i;
        if (32 * i < N)
          tc_cp_async16_zfill(st + 2 * kBfABytes + (uint32_t)(ki * kBLbo + (tok >> 3) * kTcSbo + (tok & 7) * 16),
                              xs[i] + (xbytes[i] ? koff : 0), xbytes[i]);
      }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  if (producer) {
#pragma unroll
    for (int c = 0; c < kBfStages - 1; ++c) issue(c);
  }

  const uint32_t mbar_full = (uint32_t)__cvta_generic_to_shared(&s_mbar[0]);
  const uint32_t mbar_empty = mbar_full + 8 * kBfStages;
  if (tid == 0) {
#pragma unroll
    for (int s = 0; s < kBfStages; ++s) {
      asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(mbar_full + 8 * s), "r"(kTcProducers / 32) : "memory");
      asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(mbar_empty + 8 * s) : "memory");
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"((uint32_t)__cvta_generic_to_shared(&s_tmem_base)),
                 "r"((uint32_t)kBfTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem = s_tmem_base;
  const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(N >> 3) << 17) | ((128u >> 4) << 24);

  bool failed = false;
  if (producer) {
    for (int c = 0; c < nchunks; ++c) {
      // hand step c to the MMA thread as soon as this thread's pieces of it have landed ...
      asm volatile("cp.async.wait_group %0;" ::"n"(kBfStages - 2) : "memory");
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      __syncwarp();
      if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(mbar_full + 8 * (c % kBfStages)) : "memory");
      // ... and only then wait for the stage that step c + kBfStages - 1 goes to: the MMAs of step c - 1 read it
      if (c >= 1 && c + kBfStages - 1 < nchunks &&
          !tc_mbar_wait(mbar_empty + 8 * ((c - 1) % kBfStages), (uint32_t)(((c - 1) / kBfStages) & 1))) {
        failed = true;
        break;
      }
      issue(c + kBfStages - 1);
    }
    if (!failed) {
      const int last = nchunks - 1;
      failed = !tc_mbar_wait(mbar_empty + 8 * (last % kBfStages), (uint32_t)((last / kBfStages) & 1));
    }
  } else if (lane == 0) {
    for (int c = 0; c < nchunks; ++c) {
      const int s = c % kBfStages;
      if (!tc_mbar_wait(mbar_full + 8 * s, (uint32_t)((c / kBfStages) & 1))) {
        failed = true;
        break;
      }
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint32_t a0 = sbase + (uint32_t)s * kBfStageBytes, a1 = a0 + kBfABytes, b = a1 + kBfABytes;
#pragma unroll
      for (int j = 0; j < kTcKC / 16; ++j) {
        const uint32_t acc = (c > 0 || j > 0) ? 1u : 0u;
        const uint64_t bd = tc_smem_desc(b + j * 2 * kBLbo, kBLbo, kTcSbo);
        tc_mma_f16(tmem, tc_smem_desc(a0 + j * 2 * kBfALbo, kBfALbo, kTcSbo), bd, idesc, acc);
        tc_mma_f16(tmem + NT, tc_smem_desc(a1 + j * 2 * kBfALbo, kBfALbo, kTcSbo), bd, idesc, acc);
      }
      tc_commit(mbar_empty + 8 * s);
    }
  }
  failed = __any_sync(0xffffffffu, failed);
  if (failed && lane == 0) atomicExch(&g_wgemm_tc_error, 1u);
  if (producer && !failed) tc_epilogue<SWIGLU>(a, tmem, NT, warp, lane, N, cnt, p0, row0);
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 0)
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"((uint32_t)kBfTmemCols) : "memory");
}

size_t wgemm_tc_smem_bytes() { return (size_t)kTcStages * kTcStageBytes + (size_t)kTcRing * kTcRawBytes; }

// True when the tcgen05 kernel covers this mode and shape.
bool wgemm_tc_supports(int mode, const WgArgs &args) {
  const bool swiglu = mode == WG_I4_SWIGLU || mode == WG_BF16_SWIGLU;
  const int rows_per_cta = swiglu ? 128 : 256;
  return args.R % rows_per_cta == 0 && args.K % kTcSuper == 0 && args.K / kTcKC >= kBfMinSteps;
}

int launch_wgemm_tc(int mode, const WgArgs &args, int max_tiles, cudaStream_t stream) {
  const bool swiglu = mode == WG_I4_SWIGLU || mode == WG_BF16_SWIGLU;
  dim3 grid(args.R / (swiglu ? 128 : 256), max_tiles);
  if (mode == WG_BF16_SWIGLU || mode == WG_BF16_PLAIN) {
#define BLOK_BF_LAUNCH(SW, NT)                                                                                                 \
  {                                                                                                                            \
    const size_t bsmem = (size_t)BfCfg<NT>::kStages * BfCfg<NT>::kStageBytes;                                                  \
    BLOK_CUDA(cudaFuncSetAttribute(wgemm_tc_bf16_kernel<SW, NT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bsmem));    \
    wgemm_tc_bf16_kernel<SW, NT><<<grid, kTcThreads, bsmem, stream>>>(args);                                                   \
  }
    if (args.identity_tiles) {
      grid.y = (args.n_rows + 255) / 256;
      if (swiglu) BLOK_BF_LAUNCH(true, 256) else BLOK_BF_LAUNCH(false, 256)
    } else {
      if (swiglu) BLOK_BF_LAUNCH(true, 64) else BLOK_BF_LAUNCH(false, 64)
    }
#undef BLOK_BF_LAUNCH
    return launch_status("wgemm_tc_bf16_kernel");
  }
  const size_t smem = wgemm_tc_smem_bytes();
  // tile slots: about eight rounds of CTAs (two per SM); a CTA walks the tiles of its slot
  const dim3 igrid(grid.x, std::min(max_tiles, std::max(1, 8 * 2 * sm_count() / (int)grid.x)));
  if (swiglu) {
    BLOK_CUDA(cudaFuncSetAttribute(wgemm_tc_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    wgemm_tc_kernel<true><<<igrid, kTcThreads, smem, stream>>>(args);
  } else {
    BLOK_CUDA(cudaFuncSetAttribute(wgemm_tc_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    wgemm_tc_kernel<false><<<igrid, kTcThreads, smem, stream>>>(args);
  }
  return launch_status("wgemm_tc_kernel");
}

// Non-zero once any tcgen05 GEMM CTA gave up on a barrier; cleared by the read.
int wgemm_tc_take_error(unsigned *out) {
  unsigned v = 0, zero = 0;
  BLOK_CUDA(cudaMemcpyFromSymbol(&v, g_wgemm_tc_error, sizeof(v)));
  if (v) BLOK_CUDA(cudaMemcpyToSymbol(g_wgemm_tc_error, &zero, sizeof(zero)));
  *out = v;
  return BLOK_OK;
}

}  // namespace blok
