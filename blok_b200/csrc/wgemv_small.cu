// The grouped W4A16 product for groups of a few tokens: a mat-vec-style consumer in place of the dequantising GEMM.
//
// At T = 64 tokens and 384 experts a group holds 1.8 tokens on average, and the tcgen05 kernel (wgemm_tc.cu) still turns
// every weight into a bf16 operand (about 15 thread-instructions per packed word) for a tile that is nearly empty.  Here
// the weights stream through a warp-private cp.async ring exactly as in the batch-1 decode kernel and meet the integer
// tensor-core consumer of i4_imma.cuh: a nibble becomes the byte 16 (q + 8) with one mask (unpacked ONCE per k-block),
// then every token of the group costs four mma.m16n8k32 and one post-scale.  Same arithmetic contract as
// matvec_i4_bf16_scale_k (src/kimi_exec.cu:300-323) within the floating-point bar (the error model of i4_imma.cuh);
// the SwiGLU epilogue keeps the reference's rounding points (:322, :255).
//
// One persistent CTA per SM (16 warps).  A task is (pass, 16 consecutive row-blocks), a pass being up to four tokens of
// one group (a group of 5..8 tokens is two passes over its weights): the pass's activations are quantised to block
// integers in shared memory once per task run, then each warp streams one row-block over the whole K in chunks of 14 or
// 16 k-blocks (the scales of a chunk are staged whole, as in moe_fused.cu).  Tasks are dealt out in contiguous ranges, so
// a CTA restages activations about twice per launch.  Larger groups are left to the tcgen05 kernel, which skips what this
// kernel took (WgArgs::small_max, ::small_limit) - unless they are so few (48 passes' worth) that the GEMM kernel would
// spend a CTA's whole latency, about 100 us per product, on a handful of tiles: then this kernel takes every group.
//
// Measured at T = 64 (284 groups, 7.05 GB of expert weights): gate/up and down together about 1.6 ms (4.4 TB/s); with
// every lane loading a token's operands (24 of 32 read the zero block) 1.75 ms; with a run-time token loop and pointer
// arithmetic per access 2.07 ms (164 warp instructions per 1 KB ring step against 116).
// Six tokens per pass instead of four: slower (the larger stages cost more than the second pass of the few groups of
// five or six).  The ring kept running across chunk boundaries (a second scale stage, the next chunk's scales riding
// with its first weight request): no faster (1.95 ms against 1.93 ms per layer pass; the other fifteen warps of the SM
// cover a warp's drained ring).  Four warps sharing a row-block with K split between them (better locality in HBM, but
// the CTA meets at two barriers per 14-step task): slower still (layer 2.70 ms against 2.36 ms then).
#include "i4_imma.cuh"
#include "wgemm.h"

namespace blok {

constexpr int kGsWarps = 16, kGsThreads = kGsWarps * 32;
constexpr int kGsPass = 4;                                // tokens per pass over a group's weights; a group of 5..8 takes two
constexpr int kGsDepth = 5;                               // ring steps of 1 KB (16 rows x 64 bytes) in flight per warp
constexpr int kGsMaxChunk = 16;                           // most k-blocks whose scales are staged together
constexpr int kGsScaleRow = kGsMaxChunk * 8 + 16;         // bytes per row of the scale stage (36 words: rows 4 banks apart)
constexpr int kGsWarpBytes = kGsDepth * 1024 + 16 * kGsScaleRow;
constexpr int kGsBigPasses = 48;                          // most passes of larger groups this kernel takes over from the GEMM kernel
constexpr int kGsMaxGroups = 2048;                        // small groups a launch can hold in its shared-memory list

__device__ __forceinline__ void gs_cp16(uint32_t dst, const void *src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void gs_cp16_ca(uint32_t dst, const void *src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
// Shared-memory loads by 32-bit address: the streaming loop keeps running addresses, not pointers.
__device__ __forceinline__ uint4 gs_lds128(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr) : "memory");
  return v;
}
__device__ __forceinline__ uint2 gs_lds64(uint32_t addr) {
  uint2 v;
  asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(addr) : "memory");
  return v;
}
__device__ __forceinline__ float gs_lds_bf16(uint32_t addr) {
  uint32_t v;
  asm volatile("ld.shared.u16 %0, [%1];" : "=r"(v) : "r"(addr) : "memory");
  return __uint_as_float(v << 16);
}
__device__ __forceinline__ float gs_swiglu(float g, float u) {  // :322 rounds both mat-vec outputs, :255 SiLU and the product
  g = round_bf16(g);
  u = round_bf16(u);
  return round_bf16(round_bf16(g / (1.0f + expf(-g))) * u);
}

size_t wgemv_small_smem_bytes(int K) { return (size_t)kGsPass * imma_stage_bytes(K) + (size_t)kGsWarps * kGsWarpBytes; }

// What a warp needs to stream one row-block (16 A rows: lane (g, t) holds rows g and g + 8, scale group t) over K.
struct GsStream {
  const uint4 *w_lo, *w_hi;       // this lane's 16 bytes of k-block 0 of its two rows
  const uint16_t *s_lo, *s_hi;    // scale rows of A rows 0..7 and 8..15, k-block 0
  size_t srow;                    // scales per weight row
  uint32_t ring;                  // the warp's ring, then its scale stage (shared-memory address)
  uint32_t x0, xstep;             // this lane's B operand of token 0, k-block 0, and its advance per k-block (0: the zero block)
  uint32_t meta0;                 // (f, off) of token 0, k-block 0, this lane's scale group
  uint32_t xbytes;                // bytes from one token's stage to the next
  int steps;                      // k-blocks of a row
};

// The streaming loop with the group's token count and the chunk length as compile-time constants: no per-token
// branches, the tokens' MMA chains interleave, and every address is a running value (an earlier form with run-time
// counts, pointer arithmetic per access and a division in the scale copies spent 164 warp instructions per 1 KB
// step, 42 of them integer multiply-adds for addresses, and was bound by its instruction stream at 3.4 TB/s).
template <int CNT, int CHUNK>
__device__ __forceinline__ void gs_stream(const GsStream &q, int lane, float (&acc_lo)[kGsPass], float (&acc_hi)[kGsPass]) {
  constexpr int kPieces = CHUNK / 2;  // 16-byte pieces (two k-blocks' scales) per row and chunk
  const int g = lane >> 2, t = lane & 3;
  const uint32_t ring_lane = q.ring + (uint32_t)lane * 16;
  const uint32_t sstage = q.ring + kGsDepth * 1024;
  const uint32_t sc0 = sstage + (uint32_t)(g * kGsScaleRow + t * 2);
  uint32_t xk = q.x0, mk = q.meta0;
  for (int k0 = 0; k0 < q.steps; k0 += CHUNK) {
    const int n = min(CHUNK, q.steps - k0);
    // ---- the chunk's scales, whole: 16 rows x kPieces pieces of 16 bytes ----
    __syncwarp();
#pragma unroll
    for (int i = 0; i < (16 * kPieces + 31) / 32; ++i) {
      const int pc = lane + 32 * i;
      const int row = pc / kPieces, p = pc - row * kPieces;
      if (pc < 16 * kPieces && 2 * p < n) {
        const uint16_t *src = ((row & 8) ? q.s_hi : q.s_lo) + (size_t)(row & 7) * q.srow + (size_t)(k0 + 2 * p) * 4;
        gs_cp16_ca(sstage + (uint32_t)(row * kGsScaleRow + p * 16), src);
      }
    }
    const uint4 *wl = q.w_lo + (size_t)k0 * 4, *wh = q.w_hi + (size_t)k0 * 4;  // next step to request
    uint32_t slot_in = ring_lane;
#pragma unroll
    for (int s = 0; s < kGsDepth; ++s) {
      if (s < n) {
        gs_cp16(slot_in, wl);
        gs_cp16(slot_in + 512, wh);
        wl += 4;
        wh += 4;
        slot_in += 1024;
      }
      asm volatile("cp.async.commit_group;" ::: "memory");
    }
    slot_in = ring_lane;
    uint32_t slot_out = ring_lane, sc = sc0;
    asm volatile("cp.async.wait_group %0;" ::"n"(kGsDepth - 1) : "memory");
    __syncwarp();  // the scales were copied by other lanes
    for (int s = 0; s < n; ++s) {
      asm volatile("cp.async.wait_group %0;" ::"n"(kGsDepth - 1) : "memory");
      const uint4 wlv = gs_lds128(slot_out), whv = gs_lds128(slot_out + 512);
      const float sl = gs_lds_bf16(sc), sh = gs_lds_bf16(sc + 8 * kGsScaleRow);
      uint4 x01[CNT], x23[CNT];
      uint2 meta[CNT];
#pragma unroll
      for (int tok = 0; tok < CNT; ++tok) meta[tok] = gs_lds64(mk + tok * q.xbytes);
      if (q.xstep) {  // the eight lanes that carry operands
#pragma unroll
        for (int tok = 0; tok < CNT; ++tok) {
          x01[tok] = gs_lds128(xk + tok * q.xbytes);
          x23[tok] = gs_lds128(xk + tok * q.xbytes + 16);
        }
      } else {
#pragma unroll
        for (int tok = 0; tok < CNT; ++tok) x01[tok] = x23[tok] = make_uint4(0, 0, 0, 0);
      }
      __syncwarp();
      // the A operands of the k-block's four MMAs, unpacked once for all tokens
      const uint32_t wlw[4] = {wlv.x, wlv.y, wlv.z, wlv.w}, whw[4] = {whv.x, whv.y, whv.z, whv.w};
      uint32_t a0[4], a1[4], a2[4], a3[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        a0[i] = (wlw[i] << 4) & kByteNibMask;
        a1[i] = (whw[i] << 4) & kByteNibMask;
        a2[i] = wlw[i] & kByteNibMask;
        a3[i] = whw[i] & kByteNibMask;
      }
      int d[CNT][4];
#pragma unroll
      for (int tok = 0; tok < CNT; ++tok) {
        const int noff = -(int)meta[tok].y;  // the offset 128 sum X rides in the low-limb accumulators
        d[tok][0] = 0, d[tok][1] = noff, d[tok][2] = 0, d[tok][3] = noff;
      }
#pragma unroll
      for (int i = 0; i < 4; ++i) {
#pragma unroll
        for (int tok = 0; tok < CNT; ++tok) {
          const uint32_t b0 = i == 0 ? x01[tok].x : i == 1 ? x01[tok].z : i == 2 ? x23[tok].x : x23[tok].z;
          const uint32_t b1 = i == 0 ? x01[tok].y : i == 1 ? x01[tok].w : i == 2 ? x23[tok].y : x23[tok].w;
          mma_u8s8_16832(d[tok], a0[i], a1[i], a2[i], a3[i], b0, b1);
        }
      }
#pragma unroll
      for (int tok = 0; tok < CNT; ++tok) {
        const float f = __uint_as_float(meta[tok].x);
        acc_lo[tok] = fmaf(sl, (float)(d[tok][0] * 256 + d[tok][1]) * f, acc_lo[tok]);
        acc_hi[tok] = fmaf(sh, (float)(d[tok][2] * 256 + d[tok][3]) * f, acc_hi[tok]);
      }
      // the slot just read is free: request step s + depth into it
      if (s + kGsDepth < n) {
        gs_cp16(slot_in, wl);
        gs_cp16(slot_in + 512, wh);
        wl += 4;
        wh += 4;
      }
      asm volatile("cp.async.commit_group;" ::: "memory");
      slot_out += 1024;
      if (slot_out == ring_lane + kGsDepth * 1024) slot_out = ring_lane;
      slot_in = slot_out;
      sc += 8;
      xk += q.xstep;
      mk += 32;
    }
  }
}

template <int CHUNK>
__device__ __forceinline__ void gs_stream_by_count(int cnt, const GsStream &q, int lane, float (&acc_lo)[kGsPass],
                                                   float (&acc_hi)[kGsPass]) {
  switch (cnt) {
    case 1: gs_stream<1, CHUNK>(q, lane, acc_lo, acc_hi); break;
    case 2: gs_stream<2, CHUNK>(q, lane, acc_lo, acc_hi); break;
    case 3: gs_stream<3, CHUNK>(q, lane, acc_lo, acc_hi); break;
    default: gs_stream<4, CHUNK>(q, lane, acc_lo, acc_hi); break;
  }
}

template <bool SWIGLU>
__global__ void __launch_bounds__(kGsThreads, 1) wgemv_small_kernel(const WgArgs a) {
  extern __shared__ __align__(128) unsigned char smem[];
  __shared__ unsigned short s_group[kGsMaxGroups];  // the launch's passes: tile index | pass of the tile << 12
  __shared__ int s_ngroups, s_limit;
  __shared__ int s_wcount[kGsWarps];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int K = a.K;
  const size_t xbytes = imma_stage_bytes(K);
  const uint32_t smem_addr = (uint32_t)__cvta_generic_to_shared(smem);

  // ---- which groups are this kernel's: those of up to kWgSmallTokens tokens, or every group when the larger ones are so
  // few that the GEMM kernel behind this one would spend a CTA's whole latency (about 100 us per product) on a handful
  // of tiles, while their passes here are spread over every SM (about 5 us each) ----
  const int ntiles = *a.num_tiles;
  {
    int mine = 0;
    for (int i = tid; i < ntiles; i += kGsThreads) {
      const int c = a.tile_count[i];
      if (c > kWgSmallTokens) mine += (c + kGsPass - 1) / kGsPass;
    }
    for (int o = 16; o; o >>= 1) mine += __shfl_xor_sync(0xffffffffu, mine, o);
    if (lane == 0) s_wcount[warp] = mine;
    __syncthreads();
    if (tid == 0) {
      int tot = 0;
      for (int w = 0; w < kGsWarps; ++w) tot += s_wcount[w];
      s_limit = (a.small_limit && tot <= kGsBigPasses) ? kWgTileTokens : kWgSmallTokens;
      if (a.small_limit && blockIdx.x == 0) *a.small_limit = s_limit;  // the GEMM kernel skips what this one takes
      s_ngroups = 0;
    }
    __syncthreads();
  }
  const int limit = s_limit;
  // ---- the passes in tile order, up to kGsPass tokens each (every CTA builds the same list) ----
  for (int i0 = 0; i0 < ntiles; i0 += kGsThreads) {
    const int i = i0 + tid;
    const int c = i < ntiles ? a.tile_count[i] : 0;
    const int np = (c >= 1 && c <= limit) ? (c + kGsPass - 1) / kGsPass : 0;
    // positions by a block-wide ordered count: a scan inside the warp, then the warps in order
    int incl = np;
    for (int o = 1; o < 32; o <<= 1) {
      const int v = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += v;
    }
    if (lane == 31) s_wcount[warp] = incl;
    __syncthreads();
    int pos = s_ngroups + incl - np;
    for (int w = 0; w < warp; ++w) pos += s_wcount[w];
    for (int k = 0; k < np; ++k)
      if (pos + k < kGsMaxGroups) s_group[pos + k] = (unsigned short)(i | (k << 12));
    __syncthreads();
    if (tid == 0) {
      int tot = s_ngroups;
      for (int w = 0; w < kGsWarps; ++w) tot += s_wcount[w];
      s_ngroups = min(tot, kGsMaxGroups);
    }
    __syncthreads();
  }
  const int ngroups = s_ngroups;
  const int row_blocks = SWIGLU ? a.R / 8 : a.R / 16;  // 16-row A tiles: 8 gate + 8 up rows, or 16 rows
  const int runs = (row_blocks + kGsWarps - 1) / kGsWarps;  // tasks per group
  const long total = (long)ngroups * runs;
  const long per = (total + gridDim.x - 1) / gridDim.x;
  const long q0 = (long)blockIdx.x * per, q1 = min(total, q0 + per);

  GsStream st;
  st.steps = K / 128;
  st.srow = (size_t)K / 32;
  st.xbytes = (uint32_t)xbytes;
  st.ring = smem_addr + (uint32_t)(kGsPass * xbytes) + (uint32_t)(warp * kGsWarpBytes);
  // lanes with (g >> 1) == t supply limb (g & 1) of their quad-lane's group; the others read the stage's zero block
  const bool supply = (g >> 1) == t;
  st.x0 = smem_addr + (supply ? (uint32_t)(t * 64 + (g & 1) * 32) : (uint32_t)(K * 2 + (K / 32) * 8 + 64 + (lane & 1) * 16));
  st.xstep = supply ? 256u : 0u;
  st.meta0 = smem_addr + (uint32_t)(K * 2) + (uint32_t)t * 8;
  const size_t wrow = (size_t)K / 32;  // uint4 per weight row
  const bool chunk16 = st.steps % 16 == 0;
  int staged = -1;
  for (long q = q0; q < q1; ++q) {
    const int gi = (int)(q / runs), run = (int)(q - (long)gi * runs);
    const int tile = s_group[gi] & 0xfff, tok0 = (s_group[gi] >> 12) * kGsPass;
    const int e = a.tile_expert[tile], p0 = a.tile_start[tile] + tok0, cnt = min(kGsPass, a.tile_count[tile] - tok0);
    if (gi != staged) {
      // ---- the group's activations as block integers, one stage per token ----
      __syncthreads();  // every warp is done with the previous group's stages
      for (int tok = 0; tok < cnt; ++tok) {
        const size_t xr = a.x_index ? (size_t)a.x_index[p0 + tok] : (size_t)(p0 + tok);
        const ImmaStage stg = imma_stage_carve(smem + (size_t)tok * xbytes, K);
        stage_x_imma(reinterpret_cast<const uint4 *>(a.x + xr * K), stg, K, tid, kGsThreads);
      }
      __syncthreads();
      staged = gi;
    }
    const int rb = run * kGsWarps + warp;
    if (rb >= row_blocks) continue;
    const size_t erow = (size_t)e * a.expert_stride_rows;
    const size_t r_lo = erow + (SWIGLU ? rb * 8 : rb * 16) + g;
    const size_t r_hi = SWIGLU ? r_lo : r_lo + 8;
    st.w_lo = reinterpret_cast<const uint4 *>(a.w_a) + r_lo * wrow + t;
    st.w_hi = reinterpret_cast<const uint4 *>(SWIGLU ? a.w_b : a.w_a) + r_hi * wrow + t;
    st.s_lo = a.s_a + (r_lo - g) * st.srow;
    st.s_hi = (SWIGLU ? a.s_b : a.s_a) + (r_hi - g) * st.srow;
    float acc_lo[kGsPass], acc_hi[kGsPass];
#pragma unroll
    for (int k = 0; k < kGsPass; ++k) acc_lo[k] = acc_hi[k] = 0.f;
    if (chunk16) gs_stream_by_count<16>(cnt, st, lane, acc_lo, acc_hi);
    else gs_stream_by_count<14>(cnt, st, lane, acc_lo, acc_hi);
    // ---- a row's four scale groups sit in the four lanes of its quad ----
#pragma unroll
    for (int tok = 0; tok < kGsPass; ++tok) {
      if (tok < cnt) {
        float lo = acc_lo[tok], hi = acc_hi[tok];
        lo += __shfl_xor_sync(0xffffffffu, lo, 1);
        lo += __shfl_xor_sync(0xffffffffu, lo, 2);
        hi += __shfl_xor_sync(0xffffffffu, hi, 1);
        hi += __shfl_xor_sync(0xffffffffu, hi, 2);
        const size_t p = a.out_index ? (size_t)a.out_index[p0 + tok] : (size_t)(p0 + tok);
        if (SWIGLU) {
          if (t == 0) a.out_bf16[p * a.R + rb * 8 + g] = f32_to_bf16_bits(gs_swiglu(lo, hi));
        } else if (t < 2) {
          const float v = t ? hi : lo;
          const size_t o = p * a.R + rb * 16 + g + 8 * t;
          if (a.out_f32) a.out_f32[o] = v;
          else a.out_bf16[o] = f32_to_bf16_bits(v);
        }
      }
    }
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");
}

// max_tiles: the most tiles the launch's table can hold; every pass of every tile must fit the kernel's list (two passes
// per tile of up to kWgSmallTokens tokens, kGsBigPasses more when it takes the larger groups too) and its 12-bit tile index
bool wgemv_small_supports(int mode, const WgArgs &a, int max_tiles) {
  if (max_tiles > 4096 || 2 * max_tiles + kGsBigPasses > kGsMaxGroups) return false;
  if (mode != WG_I4_SWIGLU && mode != WG_I4_PLAIN) return false;
  if (a.identity_tiles || a.K % 256 || a.R % 16) return false;  // 16-byte scale copies: an even number of k-blocks per row
  return wgemv_small_smem_bytes(a.K) <= 200 * 1024;
}

int launch_wgemv_small(int mode, const WgArgs &args, cudaStream_t stream) {
  const size_t smem = wgemv_small_smem_bytes(args.K);
  const int grid = sm_count();
  if (mode == WG_I4_SWIGLU) {
    BLOK_CUDA(cudaFuncSetAttribute(wgemv_small_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    wgemv_small_kernel<true><<<grid, kGsThreads, smem, stream>>>(args);
  } else {
    BLOK_CUDA(cudaFuncSetAttribute(wgemv_small_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    wgemv_small_kernel<false><<<grid, kGsThreads, smem, stream>>>(args);
  }
  return launch_status("wgemv_small_kernel");
}

}  // namespace blok
