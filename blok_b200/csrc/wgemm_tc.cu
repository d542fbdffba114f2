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
// count.  Per 64-column step the 128 threads (one weight row each) unpack their packed
// words into shared memory in the K-major core-matrix layout the instruction reads
// (no swizzle: 8 rows x 16 bytes per core matrix), permute the tile's activations the
// same way, and one thread issues the MMAs; tcgen05.commit on an mbarrier frees the
// stage.  The global loads of the next step are in registers while this one is
// unpacked.  Every mbarrier wait is bounded; on a timeout the CTA records an error,
// still releases its tensor memory and returns.
#include "common.cuh"
#include "wgemm.h"

namespace blok {

constexpr int kTcThreads = 128;
constexpr int kTcN = kWgTileTokens;  // token columns of a tile
constexpr int kTcKC = 64;            // weight columns per pipeline step
constexpr int kTcStages = 2;
constexpr int kTcALbo = 2048;        // bytes between core matrices adjacent in K (16 row groups x 128 B)
constexpr int kTcSbo = 128;          // bytes between 8-row groups
constexpr int kTcABytes = (kTcKC / 8) * kTcALbo;
constexpr int kTcBLbo = 1040;        // 8 token groups x 128 B, plus 16 B so that the 8 K-slices of a token hit 8 banks
constexpr int kTcBBytes = (kTcKC / 8) * kTcBLbo;
constexpr int kTcStageBytes = 2 * kTcABytes + ((kTcBBytes + 127) / 128) * 128;
constexpr int kTcTmemCols = 2 * kTcN;
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

struct TcPrefetch {
  uint4 q[2][2];    // [matrix][32-column half] packed words of this thread's row
  uint32_t sc[2];   // [matrix] the two halves' scales (bf16 pair)
  uint4 x[4];       // this thread's four 16-byte pieces of the activation tile
};

template <bool SWIGLU>
__global__ void __launch_bounds__(kTcThreads) wgemm_tc_kernel(const WgArgs a) {
  extern __shared__ __align__(128) unsigned char smem[];
  __shared__ __align__(8) unsigned long long s_mbar[kTcStages];
  __shared__ uint32_t s_tmem_base;
  const int tile = blockIdx.y;
  if (tile >= *a.num_tiles) return;
  const int tid = threadIdx.x, warp = tid >> 5;
  const int e = a.tile_expert[tile], p0 = a.tile_start[tile], cnt = a.tile_count[tile];
  const int N = max(16, (cnt + 15) & ~15);  // token columns the MMAs cover

  // ---- this thread's weight row in both 128-row blocks ----
  const int rows_per_cta = SWIGLU ? 128 : 256;
  const int row0 = blockIdx.x * rows_per_cta;
  const size_t r_a = (size_t)e * a.expert_stride_rows + row0 + tid;
  const size_t r_b = SWIGLU ? r_a : r_a + 128;
  const size_t wrow16 = (size_t)a.K / 32;  // uint4 (= scale groups) per packed row
  const uint4 *wa = reinterpret_cast<const uint4 *>(a.w_a) + r_a * wrow16;
  const uint4 *wb = reinterpret_cast<const uint4 *>(SWIGLU ? a.w_b : a.w_a) + r_b * wrow16;
  const uint32_t *sa = reinterpret_cast<const uint32_t *>(a.s_a + r_a * wrow16);
  const uint32_t *sb = reinterpret_cast<const uint32_t *>((SWIGLU ? a.s_b : a.s_a) + r_b * wrow16);
  // ---- this thread's four pieces of the activation tile: token (tid / 8) + 16 i, K-slice tid % 8 ----
  const int ki = tid & 7;
  const uint4 *xp[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int tok = (tid >> 3) + 16 * i;
    xp[i] = nullptr;
    if (tok < cnt) {
      const size_t xr = a.x_index ? (size_t)a.x_index[p0 + tok] : (size_t)(p0 + tok);
      xp[i] = reinterpret_cast<const uint4 *>(a.x + xr * a.K) + ki;
    }
  }
  auto prefetch = [&](int c, TcPrefetch &pf) {
    pf.q[0][0] = ldg_stream(wa + 2 * c);
    pf.q[0][1] = ldg_stream(wa + 2 * c + 1);
    pf.q[1][0] = ldg_stream(wb + 2 * c);
    pf.q[1][1] = ldg_stream(wb + 2 * c + 1);
    pf.sc[0] = __ldg(sa + c);
    pf.sc[1] = __ldg(sb + c);
#pragma unroll
    for (int i = 0; i < 4; ++i) pf.x[i] = xp[i] ? __ldg(xp[i] + (size_t)c * (kTcKC / 8)) : make_uint4(0, 0, 0, 0);
  };

  // ---- barriers and tensor memory ----
  const uint32_t mbar0 = (uint32_t)__cvta_generic_to_shared(&s_mbar[0]);
  const uint32_t sbase = (uint32_t)__cvta_generic_to_shared(smem);
  if (tid == 0) {
#pragma unroll
    for (int s = 0; s < kTcStages; ++s) asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(mbar0 + 8 * s) : "memory");
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"((uint32_t)__cvta_generic_to_shared(&s_tmem_base)),
                 "r"((uint32_t)kTcTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  TcPrefetch pf;
  prefetch(0, pf);
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem = s_tmem_base;
  const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(N >> 3) << 17) | ((128u >> 4) << 24);

  const int nchunks = a.K / kTcKC;
  bool failed = false;
  for (int c = 0; c < nchunks; ++c) {
    const TcPrefetch cur = pf;
    if (c + 1 < nchunks) prefetch(c + 1, pf);
    const int s = c % kTcStages;
    // the MMAs that read this stage two steps ago must be done with it
    bool ok = true;
    if (c >= kTcStages) ok = tc_mbar_wait(mbar0 + 8 * s, (uint32_t)((c / kTcStages - 1) & 1));
    if (__syncthreads_or(!ok)) {
      failed = true;
      break;
    }
    unsigned char *A0 = smem + (size_t)s * kTcStageBytes;
    unsigned char *A1 = A0 + kTcABytes;
    unsigned char *B = A1 + kTcABytes;
    const int rowoff = (tid >> 3) * kTcSbo + (tid & 7) * 16;
#pragma unroll
    for (int m = 0; m < 2; ++m) {
      unsigned char *A = m ? A1 : A0;
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const uint32_t s2 = __byte_perm(cur.sc[m], cur.sc[m], h ? 0x3232 : 0x1010);
        const uint4 q = cur.q[m][h];
        *reinterpret_cast<uint4 *>(A + (h * 4 + 0) * kTcALbo + rowoff) = tc_dequant_word(q.x, s2);
        *reinterpret_cast<uint4 *>(A + (h * 4 + 1) * kTcALbo + rowoff) = tc_dequant_word(q.y, s2);
        *reinterpret_cast<uint4 *>(A + (h * 4 + 2) * kTcALbo + rowoff) = tc_dequant_word(q.z, s2);
        *reinterpret_cast<uint4 *>(A + (h * 4 + 3) * kTcALbo + rowoff) = tc_dequant_word(q.w, s2);
      }
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      if (16 * i < N) {
        const uint4 v = cur.x[i];
        uint4 o;  // columns 0 4 1 5 2 6 3 7, as the weights
        o.x = __byte_perm(v.x, v.z, 0x5410);
        o.y = __byte_perm(v.x, v.z, 0x7632);
        o.z = __byte_perm(v.y, v.w, 0x5410);
        o.w = __byte_perm(v.y, v.w, 0x7632);
        const int tok = (tid >> 3) + 16 * i;
        *reinterpret_cast<uint4 *>(B + ki * kTcBLbo + (tok >> 3) * kTcSbo + (tok & 7) * 16) = o;
      }
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // the stores above are read by the tensor core's proxy
    __syncthreads();
    if (tid == 0) {
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint32_t a0 = sbase + (uint32_t)s * kTcStageBytes, a1 = a0 + kTcABytes, b = a1 + kTcABytes;
#pragma unroll
      for (int j = 0; j < kTcKC / 16; ++j) {
        const uint32_t acc = (c > 0 || j > 0) ? 1u : 0u;
        const uint64_t bd = tc_smem_desc(b + j * 2 * kTcBLbo, kTcBLbo, kTcSbo);
        tc_mma_f16(tmem, tc_smem_desc(a0 + j * 2 * kTcALbo, kTcALbo, kTcSbo), bd, idesc, acc);
        tc_mma_f16(tmem + kTcN, tc_smem_desc(a1 + j * 2 * kTcALbo, kTcALbo, kTcSbo), bd, idesc, acc);
      }
      tc_commit(mbar0 + 8 * s);
    }
  }

  // ---- epilogue: thread tid holds accumulator row tid of both blocks (tensor-memory lane tid) ----
  if (!failed) {
    const int last = nchunks - 1;
    const bool ok = tc_mbar_wait(mbar0 + 8 * (last % kTcStages), (uint32_t)((last / kTcStages) & 1));
    if (__syncthreads_or(!ok)) failed = true;
  }
  if (!failed) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t trow = tmem + ((uint32_t)(warp * 32) << 16);
    for (int n0 = 0; n0 < N; n0 += 16) {
      uint32_t ra[16], rb[16];
      tc_ld16(trow + n0, ra);
      tc_ld16(trow + kTcN + n0, rb);
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
            a.out_bf16[p * a.R + row0 + tid] = f32_to_bf16_bits(m);
          } else if (a.out_f32) {
            a.out_f32[p * a.R + row0 + tid] = va;
            a.out_f32[p * a.R + row0 + 128 + tid] = vb;
          } else {
            a.out_bf16[p * a.R + row0 + tid] = f32_to_bf16_bits(va);
            a.out_bf16[p * a.R + row0 + 128 + tid] = f32_to_bf16_bits(vb);
          }
        }
      }
    }
  } else if (tid == 0) {
    atomicExch(&g_wgemm_tc_error, 1u);
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 0)
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"((uint32_t)kTcTmemCols) : "memory");
}

size_t wgemm_tc_smem_bytes() { return (size_t)kTcStages * kTcStageBytes; }

// True when the tcgen05 kernel covers this mode and shape.
bool wgemm_tc_supports(int mode, const WgArgs &args) {
  if (mode != WG_I4_SWIGLU && mode != WG_I4_PLAIN) return false;
  const int rows_per_cta = mode == WG_I4_SWIGLU ? 128 : 256;
  return args.R % rows_per_cta == 0 && args.K % kTcKC == 0;
}

int launch_wgemm_tc(int mode, const WgArgs &args, int max_tiles, cudaStream_t stream) {
  const size_t smem = wgemm_tc_smem_bytes();
  const bool swiglu = mode == WG_I4_SWIGLU;
  dim3 grid(args.R / (swiglu ? 128 : 256), max_tiles);
  if (swiglu) {
    BLOK_CUDA(cudaFuncSetAttribute(wgemm_tc_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    wgemm_tc_kernel<true><<<grid, kTcThreads, smem, stream>>>(args);
  } else {
    BLOK_CUDA(cudaFuncSetAttribute(wgemm_tc_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    wgemm_tc_kernel<false><<<grid, kTcThreads, smem, stream>>>(args);
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
