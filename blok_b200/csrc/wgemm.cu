// Weight-streaming GEMM for batched tokens: out[token, row] = sum_c W[row, c] * x[token, c]
// with W either bf16 or INT4 (pack_quantized, group 32) and tokens grouped by expert.
// Used by the batched routed-MoE layer (tokens sorted by expert), the shared expert
// and the router logits at T > 8.  Reference arithmetic: matvec_i4_bf16_scale_k
// (src/kimi_exec.cu:300-323) and matvec_bf16_k (:272-284) applied per token.
//
// The weights are the large operand (9.5 GB per layer) and every selected expert's
// weights must be read once whatever the token count, so the kernel is organised
// around the weight stream ("swap-AB"): weight rows fill the M = 16 dimension of
// mma.sync.m16n8k16, tokens the N dimension.  A CTA owns 8 warps x 16 weight rows
// and one tile of up to 64 tokens of one expert; activations are staged through
// shared memory in 512-column chunks.  INT4 weights are dequantised in registers
// to the reference's exact bf16 values bf16(q * scale) (one subtract and one
// multiply on packed bf16 pairs) and reused across the tile's token columns.
#include "common.cuh"
#include "wgemm.h"
#include <algorithm>
#include <cstdlib>
#include <cstring>

namespace blok {

constexpr int kWgWarps = 8;
constexpr int kWgThreads = kWgWarps * 32;
constexpr int kWgTokens = 64;                    // tokens per tile
constexpr int kWgChunk = 512;                    // columns staged per step
constexpr int kWgTokPitch = kWgChunk * 2 + 64;   // bytes per staged token row; the 64 B skew keeps LDS.128 conflict-free

__device__ __forceinline__ uint32_t bf16x2_sub(uint32_t a, uint32_t b) {
  uint32_t r;
  asm("sub.rn.bf16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
  return r;
}
__device__ __forceinline__ uint32_t bf16x2_mul(uint32_t a, uint32_t b) {
  uint32_t r;
  asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
  return r;
}

// Exact dequantised pairs of one packed word: out[j] = (bf16(q_j * s), bf16(q_{j+4} * s)), j = 0..3.
__device__ __forceinline__ void dequant_word(uint32_t w, uint32_t s2, uint32_t (&out)[4]) {
  constexpr uint32_t kMask = 0x000f000fu, kMagic = 0x43004300u, kOff = 0x43084308u;  // 128.0 | nibble, 136.0
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    uint32_t v;
    asm("lop3.b32 %0, %1, %2, %3, 0xea;" : "=r"(v) : "r"(w >> (4 * j)), "r"(kMask), "r"(kMagic));
    out[j] = bf16x2_mul(bf16x2_sub(v, kOff), s2);
  }
}

template <int MODE>
__global__ void __launch_bounds__(kWgThreads) wgemm_kernel(const WgArgs a) {
  constexpr bool kI4 = MODE == WG_I4_SWIGLU || MODE == WG_I4_PLAIN;
  constexpr bool kSwiglu = MODE == WG_BF16_SWIGLU || MODE == WG_I4_SWIGLU;
  extern __shared__ __align__(16) unsigned char smem[];
  const int tile = blockIdx.y;
  if (tile >= *a.num_tiles) return;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int e = a.tile_expert[tile], p0 = a.tile_start[tile], cnt = a.tile_count[tile];
  if (a.small_max && cnt <= (a.small_limit ? *a.small_limit : a.small_max)) return;  // a small group: wgemv_small.cu has it
  const int ntiles = (cnt + 7) >> 3;

  // the lane's two weight rows
  const int rows_per_cta = kSwiglu ? 8 * kWgWarps : 16 * kWgWarps;
  const int row0 = blockIdx.x * rows_per_cta + (kSwiglu ? 8 : 16) * warp;
  const size_t erow = (size_t)e * a.expert_stride_rows;
  const size_t row_lo = erow + row0 + g;
  const size_t row_hi = kSwiglu ? row_lo : row_lo + 8;
  const size_t wrow16 = kI4 ? (size_t)a.K / 32 : (size_t)a.K / 8;  // uint4 per weight row
  const uint4 *w_lo = reinterpret_cast<const uint4 *>(a.w_a) + row_lo * wrow16;
  const uint4 *w_hi = reinterpret_cast<const uint4 *>(kSwiglu ? a.w_b : a.w_a) + row_hi * wrow16;
  const uint16_t *s_lo = kI4 ? a.s_a + row_lo * (a.K / 32) : nullptr;
  const uint16_t *s_hi = kI4 ? (kSwiglu ? a.s_b : a.s_a) + row_hi * (a.K / 32) : nullptr;

  float acc[8][4];
#pragma unroll
  for (int i = 0; i < 8; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;

  // K split over blockIdx.z (bf16 modes over one tile of tokens, see wgemm_splitk_factor): whole 512-column chunks
  const int kchunks = a.K / kWgChunk, nz = gridDim.z, kz = blockIdx.z;
  const int c_begin = (int)((long)kz * kchunks / nz) * kWgChunk, c_end = (int)((long)(kz + 1) * kchunks / nz) * kWgChunk;
  for (int c0 = c_begin; c0 < c_end; c0 += kWgChunk) {
    // INT4: the chunk's weights (4 k-blocks of the lane's two rows) and scales go in flight first; they do not
    // depend on the activations being staged below
    uint4 pwl[kWgChunk / 128], pwh[kWgChunk / 128];
    uint32_t psl[kWgChunk / 128], psh[kWgChunk / 128];
    if (kI4) {
#pragma unroll
      for (int kb = 0; kb < kWgChunk / 128; ++kb) {
        const int kblock = c0 / 128 + kb;
        pwl[kb] = ldg_stream(w_lo + (size_t)kblock * 4 + t);
        pwh[kb] = ldg_stream(w_hi + (size_t)kblock * 4 + t);
        psl[kb] = s_lo[kblock * 4 + t];
        psh[kb] = s_hi[kblock * 4 + t];
      }
    }
    // ---- stage the tile's activations for columns [c0, c0 + 512): 64 sixteen-byte units per token ----
    for (int u = tid; u < kWgTokens * 64; u += kWgThreads) {
      const int tok = u >> 6, unit = u & 63;
      if (tok >= 8 * ntiles) break;  // token rows beyond the tile's last 8-token group are never read
      uint4 v = make_uint4(0, 0, 0, 0);
      if (tok < cnt) {
        const int p = p0 + tok;
        const size_t xr = a.x_index ? (size_t)a.x_index[p] : (size_t)p;
        v = *reinterpret_cast<const uint4 *>(a.x + xr * a.K + c0 + unit * 8);
      }
      const int kb = unit >> 4, uu = unit & 15;
      int dst;
      if (kI4) {
        // unit uu holds columns 8uu..8uu+7 of the k-block = word i = uu&3 of quad lane tt = uu>>2;
        // pairs are re-ordered to (x0,x4)(x1,x5)(x2,x6)(x3,x7) to match one AND+OR per nibble pair
        uint4 o;
        o.x = __byte_perm(v.x, v.z, 0x5410);
        o.y = __byte_perm(v.x, v.z, 0x7632);
        o.z = __byte_perm(v.y, v.w, 0x5410);
        o.w = __byte_perm(v.y, v.w, 0x7632);
        v = o;
        dst = kb * 16 + (uu & 3) * 4 + (uu >> 2);
      } else {
        dst = unit;  // bf16 weights: lane tt's i-th load covers columns 32i + 8tt, i.e. unit 4i + tt
      }
      *reinterpret_cast<uint4 *>(smem + (size_t)tok * kWgTokPitch + dst * 16) = v;
    }
    __syncthreads();
#pragma unroll
    for (int kb = 0; kb < kWgChunk / 128; ++kb) {
      const int kblock = c0 / 128 + kb;
      uint32_t alo[4][4], ahi[4][4];  // [word i][pair j] A-fragment registers of the two rows
      if (kI4) {
        const uint32_t sl2 = psl[kb] | (psl[kb] << 16), sh2 = psh[kb] | (psh[kb] << 16);
        dequant_word(pwl[kb].x, sl2, alo[0]);
        dequant_word(pwl[kb].y, sl2, alo[1]);
        dequant_word(pwl[kb].z, sl2, alo[2]);
        dequant_word(pwl[kb].w, sl2, alo[3]);
        dequant_word(pwh[kb].x, sh2, ahi[0]);
        dequant_word(pwh[kb].y, sh2, ahi[1]);
        dequant_word(pwh[kb].z, sh2, ahi[2]);
        dequant_word(pwh[kb].w, sh2, ahi[3]);
      } else {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const uint4 wl = ldg_stream(w_lo + (size_t)kblock * 16 + i * 4 + t);
          const uint4 wh = ldg_stream(w_hi + (size_t)kblock * 16 + i * 4 + t);
          alo[i][0] = wl.x; alo[i][1] = wl.y; alo[i][2] = wl.z; alo[i][3] = wl.w;
          ahi[i][0] = wh.x; ahi[i][1] = wh.y; ahi[i][2] = wh.z; ahi[i][3] = wh.w;
        }
      }
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) {
        if (nt < ntiles) {
          const unsigned char *xt = smem + (size_t)(8 * nt + g) * kWgTokPitch + kb * 256 + t * 16;
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const uint4 xb = *reinterpret_cast<const uint4 *>(xt + i * 64);
            mma_bf16_16816(acc[nt], alo[i][0], ahi[i][0], alo[i][1], ahi[i][1], xb.x, xb.y);
            mma_bf16_16816(acc[nt], alo[i][2], ahi[i][2], alo[i][3], ahi[i][3], xb.z, xb.w);
          }
        }
      }
    }
    __syncthreads();
  }

  // ---- epilogue: lane holds rows g (acc[.][0..1]) and g+8 / up row g (acc[.][2..3]) for tokens 8nt+2t, +1 ----
#pragma unroll
  for (int nt = 0; nt < 8; ++nt) {
    if (nt >= ntiles) break;
#pragma unroll
    for (int c = 0; c < 2; ++c) {
      const int tok = 8 * nt + 2 * t + c;
      if (tok >= cnt) continue;
      if (nz > 1) {  // partial sums [split][row of x][gate rows, then up rows | rows]: the reduce kernel finishes them
        const int cols = kSwiglu ? 2 * a.R : a.R;
        float *ps = a.splitk_ws + ((size_t)kz * a.n_rows + (p0 + tok)) * cols;
        ps[row0 + g] = acc[nt][c];
        ps[(kSwiglu ? a.R : 8) + row0 + g] = acc[nt][2 + c];
        continue;
      }
      const size_t p = a.out_index ? (size_t)a.out_index[p0 + tok] : (size_t)(p0 + tok);
      if (kSwiglu) {
        float gv = round_bf16(acc[nt][c]), uv = round_bf16(acc[nt][2 + c]);
        float m = round_bf16(round_bf16(gv / (1.0f + expf(-gv))) * uv);
        a.out_bf16[p * a.R + row0 + g] = f32_to_bf16_bits(m);
      } else if (a.out_f32) {
        a.out_f32[p * a.R + row0 + g] = acc[nt][c];
        a.out_f32[p * a.R + row0 + g + 8] = acc[nt][2 + c];
      } else {
        a.out_bf16[p * a.R + row0 + g] = f32_to_bf16_bits(acc[nt][c]);
        a.out_bf16[p * a.R + row0 + g + 8] = f32_to_bf16_bits(acc[nt][2 + c]);
      }
    }
  }
}

// Adds the K-split partial sums in split order and applies the epilogue of wgemm_kernel.  grid = (ceil(R / 256), n_rows).
template <bool SWIGLU>
__global__ void wgemm_splitk_reduce_kernel(const WgArgs a, int nz) {
  const int p = blockIdx.y, row = blockIdx.x * blockDim.x + threadIdx.x;
  if (row >= a.R) return;
  const int cols = SWIGLU ? 2 * a.R : a.R;
  const float *ps = a.splitk_ws + (size_t)p * cols + row;
  const size_t stride = (size_t)a.n_rows * cols;
  float v = 0.f, u = 0.f;
  for (int z = 0; z < nz; ++z) {
    v += ps[z * stride];
    if (SWIGLU) u += ps[z * stride + a.R];
  }
  const size_t o = (a.out_index ? (size_t)a.out_index[p] : (size_t)p) * a.R + row;
  if (SWIGLU) {
    const float gv = round_bf16(v), uv = round_bf16(u);
    a.out_bf16[o] = f32_to_bf16_bits(round_bf16(round_bf16(gv / (1.0f + expf(-gv))) * uv));
  } else if (a.out_f32) {
    a.out_f32[o] = v;
  } else {
    a.out_bf16[o] = f32_to_bf16_bits(v);
  }
}

int wgemm_splitk_factor(int mode, int K, int R, int tiles) {
  if (mode != WG_BF16_PLAIN && mode != WG_BF16_SWIGLU) return 1;
  const int rows_per_cta = mode == WG_BF16_SWIGLU ? 8 * kWgWarps : 16 * kWgWarps;
  if (R % rows_per_cta || K % kWgChunk || tiles < 1) return 1;
  const int ctas = R / rows_per_cta * tiles, chunks = K / kWgChunk;
  return std::max(1, std::min(chunks, 2 * sm_count() / ctas));
}
size_t wgemm_splitk_bytes(int mode, int K, int R, int max_rows) {
  size_t worst = 0;
  {  // the weight-streaming kernel over up to kWgStreamTokens rows
    const int nz = wgemm_stream_split(mode, K, R);
    if (nz > 1) worst = (size_t)nz * std::min(max_rows, kWgStreamTokens) * (mode == WG_BF16_SWIGLU ? 2 * R : R) * sizeof(float);
  }
  for (int tiles = 1; tiles <= (max_rows + kWgTokens - 1) / kWgTokens; ++tiles) {
    const int nz = wgemm_splitk_factor(mode, K, R, tiles);
    if (nz <= 1) break;  // the factor falls as the tiles grow in number
    const size_t rows = (size_t)std::min(max_rows, tiles * kWgTokens);
    worst = std::max(worst, (size_t)nz * rows * (mode == WG_BF16_SWIGLU ? 2 * R : R) * sizeof(float));
  }
  return worst;
}

size_t wgemm_smem_bytes() { return (size_t)kWgTokens * kWgTokPitch; }

// 0 = pick by size, 1 = mma.sync kernel always, 2 = tcgen05 kernels wherever they apply
static int wgemm_forced_impl() {  // read at every launch, so that a test can switch it inside one process
  const char *e = getenv("BLOK_WGEMM_IMPL");
  if (e && strcmp(e, "mma") == 0) return 1;
  if (e && strcmp(e, "tc") == 0) return 2;
  return 0;
}

int launch_wgemm(int mode, const WgArgs &args_in, int max_tiles, cudaStream_t stream) {
  const int forced = wgemm_forced_impl();
  const bool i4 = mode == WG_I4_SWIGLU || mode == WG_I4_PLAIN;
  WgArgs args = args_in;
  {
    // groups of a few tokens first, through the mat-vec-style kernel; the kernel below then skips them
    // (not when one GEMM kernel is forced: a forced run wants every row through the same arithmetic, whatever shares
    // its group, which is what the expert-parallel parity checks compare bit for bit)
    const char *sm = getenv("BLOK_WGEMM_SMALL");
    if (i4 && forced == 0 && !(sm && sm[0] == '0') && wgemv_small_supports(mode, args, max_tiles)) {
      if (int rc = launch_wgemv_small(mode, args, stream)) return rc;
      args.small_max = kWgSmallTokens;
    }
  }
  const bool swiglu = mode == WG_BF16_SWIGLU || mode == WG_I4_SWIGLU;
  if (!i4 && forced == 0 && wgemm_stream_supports(mode, args)) {
    int nz = 1;
    if (int rc = launch_wgemm_stream(mode, args, &nz, stream)) return rc;
    if (nz > 1) {
      const dim3 rg((args.R + 255) / 256, args.n_rows);
      if (swiglu) wgemm_splitk_reduce_kernel<true><<<rg, 256, 0, stream>>>(args, nz);
      else wgemm_splitk_reduce_kernel<false><<<rg, 256, 0, stream>>>(args, nz);
      return launch_status("wgemm_splitk_reduce_kernel");
    }
    return BLOK_OK;
  }
  // bf16: the tcgen05 kernel's 256-token tiles leave most SMs idle below about 650 tokens (shared expert: 376 us from
  // 128 to 1,024 tokens, against 106 / 162 / 297 / 585 us for the K-split mma.sync kernel at 128 / 256 / 512 / 1,024)
  const bool enough = args.n_rows >= (i4 ? 256 : 640);
  if (forced != 1 && (forced == 2 || enough) && wgemm_tc_supports(mode, args)) return launch_wgemm_tc(mode, args, max_tiles, stream);
  const size_t smem = wgemm_smem_bytes();
  const int rows_per_cta = swiglu ? 8 * kWgWarps : 16 * kWgWarps;
  BLOK_REQUIRE(args.R % rows_per_cta == 0 && args.K % kWgChunk == 0, BLOK_ERR_SHAPE,
               "wgemm: rows %d must be a multiple of %d and columns %d of %d", args.R, rows_per_cta, args.K, kWgChunk);
  dim3 grid(args.R / rows_per_cta, max_tiles);
  if (!i4 && args.identity_tiles && args.splitk_ws) {
    const int nz = wgemm_splitk_factor(mode, args.K, args.R, max_tiles);
    if (nz > 1 && args.splitk_bytes >= (size_t)nz * args.n_rows * (swiglu ? 2 * args.R : args.R) * sizeof(float)) grid.z = nz;
  }
#define BLOK_WG_LAUNCH(M)                                                                                         \
  {                                                                                                                \
    BLOK_CUDA(cudaFuncSetAttribute(wgemm_kernel<M>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));      \
    wgemm_kernel<M><<<grid, kWgThreads, smem, stream>>>(args);                                                     \
  }
  switch (mode) {
    case WG_BF16_PLAIN: BLOK_WG_LAUNCH(WG_BF16_PLAIN) break;
    case WG_BF16_SWIGLU: BLOK_WG_LAUNCH(WG_BF16_SWIGLU) break;
    case WG_I4_SWIGLU: BLOK_WG_LAUNCH(WG_I4_SWIGLU) break;
    default: BLOK_WG_LAUNCH(WG_I4_PLAIN) break;
  }
#undef BLOK_WG_LAUNCH
  if (int rc = launch_status("wgemm_kernel")) return rc;
  if (grid.z > 1) {
    const dim3 rg((args.R + 255) / 256, args.n_rows);
    if (swiglu) wgemm_splitk_reduce_kernel<true><<<rg, 256, 0, stream>>>(args, (int)grid.z);
    else wgemm_splitk_reduce_kernel<false><<<rg, 256, 0, stream>>>(args, (int)grid.z);
    return launch_status("wgemm_splitk_reduce_kernel");
  }
  return BLOK_OK;
}

int launch_wgemm_rows(int mode, const void *w_a, const void *w_b, const uint16_t *x, uint16_t *out_bf16, float *out_f32, int R, int K,
                      int T, float *splitk_ws, size_t splitk_bytes, cudaStream_t stream) {
  WgArgs r;
  r.w_a = w_a; r.w_b = w_b; r.s_a = r.s_b = nullptr; r.expert_stride_rows = 0; r.x = x; r.x_index = nullptr;
  r.K = K; r.R = R; r.out_bf16 = out_bf16; r.out_f32 = out_f32;
  r.tile_expert = r.tile_start = r.tile_count = r.num_tiles = nullptr; r.out_index = nullptr;
  r.identity_tiles = 1; r.n_rows = T; r.splitk_ws = splitk_ws; r.splitk_bytes = splitk_bytes;
  BLOK_REQUIRE(wgemm_stream_supports(mode, r), BLOK_ERR_SHAPE, "wgemm rows: %d rows x %d columns over %d tokens is outside the streaming kernel",
               R, K, T);
  int nz = 1;
  if (int rc = launch_wgemm_stream(mode, r, &nz, stream)) return rc;
  if (nz > 1) {
    const dim3 rg((R + 255) / 256, T);
    if (mode == WG_BF16_SWIGLU) wgemm_splitk_reduce_kernel<true><<<rg, 256, 0, stream>>>(r, nz);
    else wgemm_splitk_reduce_kernel<false><<<rg, 256, 0, stream>>>(r, nz);
    return launch_status("wgemm_splitk_reduce_kernel");
  }
  return BLOK_OK;
}

}  // namespace blok
