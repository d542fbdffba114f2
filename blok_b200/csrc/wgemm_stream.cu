// bf16 weights against 9 to 64 rows of activations (a decode step of 9..64 sequences, a rank's share of a small batch):
//   out[token, row] = sum_c W[row, c] * x[token, c]          (matvec_bf16_k, src/kimi_exec.cu:272-284, per token)
// with the SwiGLU front half as an option (gate and up rows of the same index, :255, :674-686).
//
// At these counts the product is bound by the weight stream, not by the tensor cores, and the kernel is built as the
// batch-1 kernels are: every warp owns 16 weight rows (8 gate + 8 up rows) and pulls them through a private ring of
// 1 KB steps (16 rows x 64 bytes, cp.async, kStDepth steps in flight), so that a CTA of eight warps keeps 64 KB of
// requests outstanding whatever the consumers do.  The activations of the CTA's K-range reach shared memory in chunks
// of 256 columns, double buffered with cp.async (the copy of chunk c + 1 rides with the weight requests of chunk c),
// one CTA-wide barrier per chunk.  A ring step feeds two mma.sync.m16n8k16 per group of 8 tokens.
//
// The mma.sync GEMM (wgemm.cu) loads a k-block's weights right before it uses them and stages the activations
// between two barriers; over one tile of tokens it reached 0.7-0.8 TB/s (the four projections of the attention block
// at 32 sequences: 76 us each; the vocabulary projection ran 8 rows at a time, four passes over its 2.35 GB).
//
// Matrices with few rows are split over K (blockIdx.y) so that about two CTAs per SM run; the partial sums go to the
// caller's scratch in the layout of wgemm_splitk_reduce_kernel, which adds them in split order.
#include <algorithm>

#include "bf16_mma.cuh"
#include "wgemm.h"

namespace blok {

constexpr int kStDepth = 8;                      // ring steps of 1 KB in flight per warp
constexpr int kStChunk = 256;                    // columns of the activations per buffer (8 ring steps)
constexpr int kStPitch = kStChunk * 2 + 64;      // bytes per staged token row: two rows of a quarter-warp hit all banks
constexpr int kStMaxWarps = 8;

__device__ __forceinline__ void st_cp16(uint32_t dst, const void *src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ uint4 st_lds128(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr) : "memory");
  return v;
}

// NT = groups of 8 tokens the launch covers (n_rows <= 8 NT).  blockDim.x / 32 warps, each 16 rows (SWIGLU: 8 + 8).
template <int NT, bool SWIGLU>
__global__ void __launch_bounds__(kStMaxWarps * 32) wgemm_stream_kernel(const WgArgs a) {
  extern __shared__ __align__(128) unsigned char smem[];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarps = blockDim.x >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int T = a.n_rows, K = a.K;
  const int row0 = (blockIdx.x * nwarps + warp) * (SWIGLU ? 8 : 16);
  const size_t wrow = (size_t)K / 8;  // uint4 per weight row
  // whole 256-column chunks of K per split
  const int chunks = K / kStChunk, nz = gridDim.y, kz = blockIdx.y;
  const int c_begin = (int)((long)kz * chunks / nz), c_end = (int)((long)(kz + 1) * chunks / nz);
  const int nchunks = c_end - c_begin, nsteps = nchunks * (kStChunk / 32);
  const uint4 *w_lo = reinterpret_cast<const uint4 *>(a.w_a) + (size_t)(row0 + g) * wrow + (size_t)c_begin * (kStChunk / 8) + t;
  const uint4 *w_hi = SWIGLU ? reinterpret_cast<const uint4 *>(a.w_b) + (size_t)(row0 + g) * wrow + (size_t)c_begin * (kStChunk / 8) + t
                             : w_lo + 8 * wrow;
  const uint32_t sbase = (uint32_t)__cvta_generic_to_shared(smem);
  constexpr uint32_t kBufBytes = 8 * NT * kStPitch;
  const uint32_t ring_lane = sbase + 2 * kBufBytes + (uint32_t)warp * (kStDepth * 1024) + (uint32_t)lane * 16;

  // the CTA's copy of chunk c of the activations (tokens past the last repeat it: their columns of D are never stored)
  auto stage = [&](int c, int buf) {
    const uint32_t dst = sbase + (uint32_t)buf * kBufBytes;
    for (int u = tid; u < 8 * NT * 32; u += blockDim.x) {
      const int tok = u >> 5, unit = u & 31;
      const int src_tok = tok < T ? tok : T - 1;
      st_cp16(dst + (uint32_t)(tok * kStPitch + unit * 16), a.x + (size_t)src_tok * K + (size_t)c * kStChunk + unit * 8);
    }
  };

  float acc[NT][4];
#pragma unroll
  for (int i = 0; i < NT; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;

  if (nchunks > 0) stage(c_begin, 0);
  const uint4 *wl = w_lo, *wh = w_hi;  // next ring step to request
  {
    uint32_t slot = ring_lane;
#pragma unroll
    for (int s = 0; s < kStDepth; ++s) {
      if (s < nsteps) {
        st_cp16(slot, wl);
        st_cp16(slot + 512, wh);
        wl += 4;
        wh += 4;
        slot += 1024;
      }
      asm volatile("cp.async.commit_group;" ::: "memory");
    }
  }
  uint32_t slot = ring_lane;
  int requested = kStDepth;
  // this lane's activation fragment of token g of group 0, k-step 0 of a buffer
  const uint32_t xlane = sbase + (uint32_t)(g * kStPitch + t * 16);
  for (int ci = 0; ci < nchunks; ++ci) {
    // the chunk's activations were committed at least kStDepth groups ago (with the first ring step of the chunk
    // before): complete for this thread after the wait, for the CTA after the barrier, which also frees the other buffer
    asm volatile("cp.async.wait_group %0;" ::"n"(kStDepth - 1) : "memory");
    __syncthreads();
    if (ci + 1 < nchunks) stage(c_begin + ci + 1, (ci + 1) & 1);
    uint32_t xs = xlane + (uint32_t)(ci & 1) * kBufBytes;
#pragma unroll 2
    for (int s = 0; s < kStChunk / 32; ++s) {
      asm volatile("cp.async.wait_group %0;" ::"n"(kStDepth - 1) : "memory");
      const uint4 wlv = st_lds128(slot), whv = st_lds128(slot + 512);
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        const uint4 xb = st_lds128(xs + (uint32_t)(nt * 8 * kStPitch));
        mma_bf16_16816(acc[nt], wlv.x, whv.x, wlv.y, whv.y, xb.x, xb.y);
        mma_bf16_16816(acc[nt], wlv.z, whv.z, wlv.w, whv.w, xb.z, xb.w);
      }
      if (requested < nsteps) {  // the slot just read takes the step a ring's depth ahead
        st_cp16(slot, wl);
        st_cp16(slot + 512, wh);
        wl += 4;
        wh += 4;
      }
      ++requested;
      asm volatile("cp.async.commit_group;" ::: "memory");
      slot += 1024;
      if (slot == ring_lane + kStDepth * 1024) slot = ring_lane;
      xs += 64;
    }
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");

  // ---- epilogue: the lane holds rows g (acc[.][0..1]) and g + 8 / up row g (acc[.][2..3]) of tokens 8 nt + 2 t, + 1 ----
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
    for (int c = 0; c < 2; ++c) {
      const int tok = 8 * nt + 2 * t + c;
      if (tok >= T) continue;
      if (nz > 1) {  // [split][token][gate rows, then up rows | rows], as wgemm_splitk_reduce_kernel reads it
        const int cols = SWIGLU ? 2 * a.R : a.R;
        float *ps = a.splitk_ws + ((size_t)kz * T + tok) * cols;
        ps[row0 + g] = acc[nt][c];
        ps[(SWIGLU ? a.R : 8) + row0 + g] = acc[nt][2 + c];
        continue;
      }
      const size_t o = (size_t)tok * a.R + row0 + g;
      if (SWIGLU) {
        const float gv = round_bf16(acc[nt][c]), uv = round_bf16(acc[nt][2 + c]);
        a.out_bf16[o] = f32_to_bf16_bits(round_bf16(round_bf16(gv / (1.0f + expf(-gv))) * uv));
      } else if (a.out_f32) {
        a.out_f32[o] = acc[nt][c];
        a.out_f32[o + 8] = acc[nt][2 + c];
      } else {
        a.out_bf16[o] = f32_to_bf16_bits(acc[nt][c]);
        a.out_bf16[o + 8] = f32_to_bf16_bits(acc[nt][2 + c]);
      }
    }
  }
}

static bool st_aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

bool wgemm_stream_supports(int mode, const WgArgs &a) {
  if (mode != WG_BF16_PLAIN && mode != WG_BF16_SWIGLU) return false;
  if (!a.identity_tiles || a.n_rows < 1 || a.n_rows > kWgStreamTokens || a.x_index || a.out_index) return false;
  if (a.K % kStChunk || a.R % (mode == WG_BF16_SWIGLU ? 8 : 16)) return false;
  return st_aligned16(a.w_a) && st_aligned16(a.x) && (mode != WG_BF16_SWIGLU || st_aligned16(a.w_b));
}

// Warps per CTA (a CTA of w warps covers 16 w rows, or 8 w gate + 8 w up rows): as many as divide the rows while the
// K-split can still give every SM a CTA; a wide CTA shares one copy of the activations among more weight rows.
static int st_warps(int mode, int K, int R) {
  const int blocks = R / (mode == WG_BF16_SWIGLU ? 8 : 16);  // one per warp
  const int max_split = std::max(1, K / kStChunk / 2);
  for (int w = kStMaxWarps; w > 1; w >>= 1)
    if (blocks % w == 0 && (long)(blocks / w) * max_split >= sm_count()) return w;
  for (int w = kStMaxWarps; w > 1; w >>= 1)
    if (blocks % w == 0) return w;
  return 1;
}

int wgemm_stream_split(int mode, int K, int R) {
  if ((mode != WG_BF16_PLAIN && mode != WG_BF16_SWIGLU) || K % kStChunk || R % (mode == WG_BF16_SWIGLU ? 8 : 16)) return 1;
  const int ctas = R / (mode == WG_BF16_SWIGLU ? 8 : 16) / st_warps(mode, K, R), chunks = K / kStChunk;
  return std::max(1, std::min(chunks / 2, 2 * sm_count() / ctas));  // at least two chunks per split
}

// Launches the kernel; *splits = the K-split it used (> 1: the partial sums wait in args.splitk_ws for the reduce kernel).
int launch_wgemm_stream(int mode, const WgArgs &args, int *splits, cudaStream_t stream) {
  const bool swiglu = mode == WG_BF16_SWIGLU;
  const int warps = st_warps(mode, args.K, args.R);
  int nz = wgemm_stream_split(mode, args.K, args.R);
  const size_t per_split = (size_t)args.n_rows * (swiglu ? 2 * args.R : args.R) * sizeof(float);
  if (nz > 1 && (!args.splitk_ws || args.splitk_bytes < per_split * nz)) nz = args.splitk_ws ? (int)std::max<size_t>(1, args.splitk_bytes / per_split) : 1;
  const int nt = args.n_rows <= 16 ? 2 : (args.n_rows <= 32 ? 4 : 8);
  const size_t smem = (size_t)2 * 8 * nt * kStPitch + (size_t)warps * kStDepth * 1024;
  const dim3 grid(args.R / (swiglu ? 8 : 16) / warps, nz);
#define BLOK_ST_LAUNCH(NT, SW)                                                                                          \
  {                                                                                                                     \
    BLOK_CUDA(cudaFuncSetAttribute(wgemm_stream_kernel<NT, SW>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); \
    wgemm_stream_kernel<NT, SW><<<grid, warps * 32, smem, stream>>>(args);                                              \
  }
  if (swiglu) {
    if (nt == 2) BLOK_ST_LAUNCH(2, true) else if (nt == 4) BLOK_ST_LAUNCH(4, true) else BLOK_ST_LAUNCH(8, true)
  } else {
    if (nt == 2) BLOK_ST_LAUNCH(2, false) else if (nt == 4) BLOK_ST_LAUNCH(4, false) else BLOK_ST_LAUNCH(8, false)
  }
#undef BLOK_ST_LAUNCH
  *splits = nz;
  return launch_status("wgemm_stream_kernel");
}

}  // namespace blok
