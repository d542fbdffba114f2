// The grouped W4A16 product for groups of up to four tokens: a mat-vec-style consumer in place of the dequantising GEMM.
//
// At T = 64 tokens and 384 experts a group holds 1.8 tokens on average, and the tcgen05 kernel (wgemm_tc.cu) still turns
// every weight into a bf16 operand (about 15 thread-instructions per packed word) for a tile that is nearly empty.  Here
// the weights stream through a warp-private cp.async ring exactly as in the batch-1 decode kernel and meet the integer
// tensor-core consumer of i4_imma.cuh: a nibble becomes the byte 16 (q + 8) with one mask (unpacked ONCE per k-block),
// then every token of the group costs four mma.m16n8k32 and one post-scale.  Same arithmetic contract as
// matvec_i4_bf16_scale_k (src/kimi_exec.cu:300-323) within the floating-point bar (the error model of i4_imma.cuh);
// the SwiGLU epilogue keeps the reference's rounding points (:322, :255).
//
// One persistent CTA per SM (16 warps).  A task is (group, 16 consecutive row-blocks): the group's activations are
// quantised to block integers in shared memory once per task run, then each warp streams one row-block over the whole
// K in chunks of 14 k-blocks (the scales of a chunk are staged whole, as in moe_fused.cu).  Tasks are numbered over the
// launch's small groups only and dealt out in contiguous ranges, so a CTA restages activations about twice per launch.
// Groups of more than four tokens are left to the tcgen05 kernel, which skips the small ones (WgArgs::small_max).
//
// Measured at T = 64 (284 groups, 7.05 GB of expert weights): gate/up 1.35 ms, down 0.72 ms (3.3-3.5 TB/s), the same
// rate as the tcgen05 kernel on these nearly empty tiles.  Six tokens per group instead of four: slower (gate/up
// 1.54 ms; the few groups of five or six cost the tcgen05 kernel less than the larger stages cost this one).  Four
// warps sharing a row-block with K split between them (better locality in HBM, but the CTA meets at two barriers per
// 14-step task): slower still (layer 2.70 ms against 2.36 ms).
#include "i4_imma.cuh"
#include "wgemm.h"

namespace blok {

constexpr int kGsWarps = 16, kGsThreads = kGsWarps * 32;
constexpr int kGsDepth = 5;                               // ring steps of 1 KB (16 rows x 64 bytes) in flight per warp
constexpr int kGsChunk = 14;                              // k-blocks whose scales are staged together
constexpr int kGsScaleRow = 16 * 8 + 8;                   // bytes per row of the scale stage (odd multiple of 8: all banks)
constexpr int kGsWarpBytes = kGsDepth * 1024 + 16 * kGsScaleRow;
constexpr int kGsMaxGroups = 2048;                        // small groups a launch can hold in its shared-memory list

__device__ __forceinline__ void gs_cp16(uint32_t dst, const void *src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void gs_cp8(uint32_t dst, const void *src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ float gs_swiglu(float g, float u) {  // :322 rounds both mat-vec outputs, :255 SiLU and the product
  g = round_bf16(g);
  u = round_bf16(u);
  return round_bf16(round_bf16(g / (1.0f + expf(-g))) * u);
}

size_t wgemv_small_smem_bytes(int K) { return (size_t)kWgSmallTokens * imma_stage_bytes(K) + (size_t)kGsWarps * kGsWarpBytes; }

template <bool SWIGLU>
__global__ void __launch_bounds__(kGsThreads, 1) wgemv_small_kernel(const WgArgs a) {
  extern __shared__ __align__(128) unsigned char smem[];
  __shared__ int s_group[kGsMaxGroups];  // tile indices of the launch's small groups
  __shared__ int s_ngroups;
  __shared__ int s_wcount[kGsWarps];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int K = a.K;
  const size_t xbytes = imma_stage_bytes(K);
  unsigned char *ring_ptr = smem + (size_t)kWgSmallTokens * xbytes + (size_t)warp * kGsWarpBytes;
  const uint32_t ring = (uint32_t)__cvta_generic_to_shared(ring_ptr);

  // ---- the launch's small groups, in tile order (every CTA builds the same list) ----
  if (tid == 0) s_ngroups = 0;
  __syncthreads();
  const int ntiles = *a.num_tiles;
  for (int i0 = 0; i0 < ntiles; i0 += kGsThreads) {
    const int i = i0 + tid;
    const bool small = i < ntiles && a.tile_count[i] >= 1 && a.tile_count[i] <= kWgSmallTokens;
    // positions by a block-wide ordered count: ballot per warp, then the warps in order
    const unsigned m = __ballot_sync(0xffffffffu, small);
    if (lane == 0) s_wcount[warp] = __popc(m);
    __syncthreads();
    int base = s_ngroups;
    for (int w = 0; w < warp; ++w) base += s_wcount[w];
    if (small) {
      const int pos = base + __popc(m & ((1u << lane) - 1u));
      if (pos < kGsMaxGroups) s_group[pos] = i;
    }
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

  const int steps = K / 128;  // k-blocks of a row
  const size_t wrow = (size_t)K / 32, srow = (size_t)K / 32;  // uint4 per weight row, scales per row
  const bool supply = (g >> 1) == t;
  int staged = -1;
  for (long q = q0; q < q1; ++q) {
    const int gi = (int)(q / runs), run = (int)(q - (long)gi * runs);
    const int tile = s_group[gi];
    const int e = a.tile_expert[tile], p0 = a.tile_start[tile], cnt = a.tile_count[tile];
    if (gi != staged) {
      // ---- the group's activations as block integers, one stage per token ----
      __syncthreads();  // every warp is done with the previous group's stages
      for (int tok = 0; tok < cnt; ++tok) {
        const size_t xr = a.x_index ? (size_t)a.x_index[p0 + tok] : (size_t)(p0 + tok);
        const ImmaStage st = imma_stage_carve(smem + (size_t)tok * xbytes, K);
        stage_x_imma(reinterpret_cast<const uint4 *>(a.x + xr * K), st, K, tid, kGsThreads);
      }
      __syncthreads();
      staged = gi;
    }
    const int rb = run * kGsWarps + warp;
    if (rb >= row_blocks) continue;
    const size_t erow = (size_t)e * a.expert_stride_rows;
    const size_t r_lo = erow + (SWIGLU ? rb * 8 : rb * 16) + g;
    const size_t r_hi = SWIGLU ? r_lo : r_lo + 8;
    const uint4 *w_lo = reinterpret_cast<const uint4 *>(a.w_a) + r_lo * wrow + t;
    const uint4 *w_hi = reinterpret_cast<const uint4 *>(SWIGLU ? a.w_b : a.w_a) + r_hi * wrow + t;
    const uint16_t *s_lo = a.s_a + (r_lo - g) * srow;                    // scale rows of A rows 0..7
    const uint16_t *s_hi = (SWIGLU ? a.s_b : a.s_a) + (r_hi - g) * srow;  // ... and 8..15
    float acc_lo[kWgSmallTokens], acc_hi[kWgSmallTokens];
#pragma unroll
    for (int k = 0; k < kWgSmallTokens; ++k) acc_lo[k] = acc_hi[k] = 0.f;
    const unsigned char *sc_lo = ring_ptr + kGsDepth * 1024 + g * kGsScaleRow + t * 2;
    const unsigned char *sc_hi = sc_lo + 8 * kGsScaleRow;
    for (int k0 = 0; k0 < steps; k0 += kGsChunk) {
      const int n = min(kGsChunk, steps - k0);
      // the chunk's scales, whole (consecutive lanes copy consecutive 8-byte pieces of a row), then the first steps
      __syncwarp();
      for (int pc = lane; pc < 16 * n; pc += 32) {
        const int row = pc / n, s = pc - row * n;
        const uint16_t *src = ((row & 8) ? s_hi : s_lo) + (size_t)(row & 7) * srow + (size_t)(k0 + s) * 4;
        gs_cp8(ring + kGsDepth * 1024 + (uint32_t)(row * kGsScaleRow + s * 8), src);
      }
      auto issue = [&](int s) {
        if (s < n) {
          const uint32_t base = ring + (uint32_t)(s % kGsDepth) * 1024 + (uint32_t)lane * 16;
          gs_cp16(base, w_lo + (size_t)(k0 + s) * 4);
          gs_cp16(base + 512, w_hi + (size_t)(k0 + s) * 4);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
      };
#pragma unroll
      for (int s = 0; s < kGsDepth; ++s) issue(s);
      for (int s = 0; s < n; ++s) {
        asm volatile("cp.async.wait_group %0;" ::"n"(kGsDepth - 1) : "memory");
        if (s == 0) __syncwarp();  // the scales were copied by other lanes
        const unsigned char *slot = ring_ptr + (size_t)(s % kGsDepth) * 1024;
        const uint4 wl = *reinterpret_cast<const uint4 *>(slot + lane * 16);
        const uint4 wh = *reinterpret_cast<const uint4 *>(slot + 512 + lane * 16);
        const float sl = bf16_bits_to_f32(*reinterpret_cast<const uint16_t *>(sc_lo + s * 8));
        const float sh = bf16_bits_to_f32(*reinterpret_cast<const uint16_t *>(sc_hi + s * 8));
        // the A operands of the k-block's four MMAs, unpacked once for all tokens
        const uint32_t wlw[4] = {wl.x, wl.y, wl.z, wl.w}, whw[4] = {wh.x, wh.y, wh.z, wh.w};
        uint32_t a0[4], a1[4], a2[4], a3[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          a0[i] = (wlw[i] << 4) & kByteNibMask;
          a1[i] = (whw[i] << 4) & kByteNibMask;
          a2[i] = wlw[i] & kByteNibMask;
          a3[i] = whw[i] & kByteNibMask;
        }
        const int kb = k0 + s;
#pragma unroll
        for (int tok = 0; tok < kWgSmallTokens; ++tok) {
          if (tok < cnt) {
            const unsigned char *xs = smem + (size_t)tok * xbytes;
            const uint4 *xp = supply ? reinterpret_cast<const uint4 *>(xs + (size_t)kb * 256 + t * 64 + (g & 1) * 32)
                                     : reinterpret_cast<const uint4 *>(xs + (size_t)K * 2 + (size_t)(K / 32) * 8) + 4 + (lane & 1);
            const uint4 x01 = xp[0], x23 = xp[1];
            int d[4] = {0, 0, 0, 0};
            mma_u8s8_16832(d, a0[0], a1[0], a2[0], a3[0], x01.x, x01.y);
            mma_u8s8_16832(d, a0[1], a1[1], a2[1], a3[1], x01.z, x01.w);
            mma_u8s8_16832(d, a0[2], a1[2], a2[2], a3[2], x23.x, x23.y);
            mma_u8s8_16832(d, a0[3], a1[3], a2[3], a3[3], x23.z, x23.w);
            const uint2 meta = reinterpret_cast<const uint2 *>(xs + (size_t)K * 2)[kb * 4 + t];
            imma_post(d, meta, sl, sh, acc_lo[tok], acc_hi[tok]);
          }
        }
        issue(s + kGsDepth);
      }
    }
    // ---- a row's four scale groups sit in the four lanes of its quad ----
#pragma unroll
    for (int tok = 0; tok < kWgSmallTokens; ++tok) {
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

bool wgemv_small_supports(int mode, const WgArgs &a) {
  if (mode != WG_I4_SWIGLU && mode != WG_I4_PLAIN) return false;
  if (a.identity_tiles || a.K % 128 || a.R % 16) return false;
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
