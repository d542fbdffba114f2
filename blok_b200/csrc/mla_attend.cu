// The attention core of absorbed MLA decode: one pass over the bf16 latent cache
// with an online softmax on mma.sync tensor cores (flash-decoding, split over the
// sequence).  Replaces attn_tile_score_k / max / sum / accum (src/kimi_exec.cu:414-475).
//
// All 64 heads of a sequence share one latent row per token (multi-query shape):
// per token 1,152 B are read once and feed 64 x (576 + 512) multiply-adds, 121
// flop/B.  A CTA owns one (sequence, token range); per 32-token tile
//   S[64 x 32]  = Q[64 x 576] . K^T          16 warps: 4 head groups x 4 token octets
//   online softmax per head row (running max and sum in registers)
//   O[64 x 512] += P[64 x 32] . C[32 x 512]  16 warps: 4 head groups x 4 latent quarters
// Q and two K/V tiles live in shared memory (cp.async double buffer); P is passed
// between the two warp layouts through shared memory.
#include "common.cuh"

namespace blok {

constexpr int kAttHeads = 64, kAttD = 576, kAttDV = 512;
constexpr int kAttTile = 32;
constexpr int kAttWarps = 16, kAttThreads = kAttWarps * 32;
constexpr int kAttPitch = kAttD * 2 + 16;  // bytes per staged row: 16 B of skew keeps ldmatrix conflict-free
constexpr int kAttSPitch = 36;             // floats per row of the score tile

__device__ __forceinline__ void att_cp16(uint32_t dst, const void *src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t &r0, uint32_t &r1, uint32_t &r2, uint32_t &r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t addr, uint32_t &r0, uint32_t &r1, uint32_t &r2, uint32_t &r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}

size_t mla_attend_smem_bytes() {
  return (size_t)kAttHeads * kAttPitch + 2 * (size_t)kAttTile * kAttPitch + (size_t)kAttHeads * kAttSPitch * 4;
}

// grid = (splits, B).  part_o fp32 [B, splits, 64, 512] (unnormalised), part_ml fp32 [B, splits, 64, 2].
// Dense cache: sequence b's rows start at cache + b * ctx_stride rows (ctx_stride 0: every b reads the same rows, the
// tokens of one prefill chunk).  PAGED: cache is a pool of pages of page_rows rows (a multiple of the 32-row tile, so
// a tile never straddles two pages); row t of sequence b lives in page block_table[slot * table_stride + t / page_rows]
// with slot = slot_of[b] (b itself when slot_of is null).
template <bool PAGED>
__global__ void __launch_bounds__(kAttThreads, 1)
    mla_attend_kernel(const uint16_t *__restrict__ q, const uint16_t *__restrict__ cache, long ctx_stride,
                      const int *__restrict__ seq_len, float scale, float *__restrict__ part_o,
                      float *__restrict__ part_ml, const int *__restrict__ block_table, const int *__restrict__ slot_of,
                      int table_stride, int page_rows) {
  extern __shared__ __align__(16) unsigned char smem[];
  unsigned char *Qs = smem;
  unsigned char *KVs = Qs + (size_t)kAttHeads * kAttPitch;
  float *Ss = reinterpret_cast<float *>(KVs + 2 * (size_t)kAttTile * kAttPitch);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int hg = warp & 3, lq = warp >> 2;
  const int split = blockIdx.x, splits = gridDim.x, b = blockIdx.y;
  const int seq = seq_len[b];
  const int ntiles = (seq + kAttTile - 1) / kAttTile;
  const int per = (ntiles + splits - 1) / splits;
  const int ts = split * per, te = min(ntiles, ts + per);
  float *my_ml = part_ml + ((size_t)b * splits + split) * kAttHeads * 2;
  if (ts >= te) {  // nothing to do for this split: mark it empty for the merge
    if (tid < kAttHeads) {
      my_ml[tid * 2] = -INFINITY;
      my_ml[tid * 2 + 1] = 0.f;
    }
    return;
  }
  const uint32_t Qs_a = (uint32_t)__cvta_generic_to_shared(Qs);
  const uint32_t KVs_a = (uint32_t)__cvta_generic_to_shared(KVs);
  const uint16_t *cache_b = PAGED ? cache : cache + (size_t)b * ctx_stride * kAttD;
  const int *table_b = PAGED ? block_table + (size_t)(slot_of ? slot_of[b] : b) * table_stride : nullptr;

  auto load_tile = [&](int tile, int buf) {
    constexpr int per_row = kAttD * 2 / 16;  // 72 uint4 per row
    const uint16_t *base = cache_b;
    int first = 0;  // the row of `base` that holds the tile's first token
    if (PAGED) {
      const int t0 = tile * kAttTile;
      base = cache + (size_t)table_b[t0 / page_rows] * page_rows * kAttD;
      first = t0 % page_rows - t0;
    }
    for (int u = tid; u < kAttTile * per_row; u += kAttThreads) {
      int r = u / per_row, c = u - r * per_row;
      int tok = min(tile * kAttTile + r, seq - 1);  // rows past the end repeat the last token; they are masked
      att_cp16(KVs_a + (uint32_t)(buf * kAttTile + r) * kAttPitch + c * 16, base + (size_t)(tok + first) * kAttD + c * 8);
    }
  };
  {
    constexpr int per_row = kAttD * 2 / 16;
    const uint16_t *qb = q + (size_t)b * kAttHeads * kAttD;
    for (int u = tid; u < kAttHeads * per_row; u += kAttThreads) {
      int r = u / per_row, c = u - r * per_row;
      att_cp16(Qs_a + (uint32_t)r * kAttPitch + c * 16, qb + (size_t)r * kAttD + c * 8);
    }
  }
  load_tile(ts, 0);
  asm volatile("cp.async.commit_group;" ::: "memory");

  float o[16][4];
#pragma unroll
  for (int j = 0; j < 16; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;
  float m_lo = -INFINITY, m_hi = -INFINITY, l_lo = 0.f, l_hi = 0.f;

  for (int tile = ts; tile < te; ++tile) {
    const int buf = (tile - ts) & 1;
    if (tile + 1 < te) load_tile(tile + 1, buf ^ 1);
    asm volatile("cp.async.commit_group;" ::: "memory");
    asm volatile("cp.async.wait_group 1;" ::: "memory");
    __syncthreads();

    // ---- S = Q K^T for heads [16hg, +16) x tokens [8lq, +8) of the tile -----------------------
    {
      float s[4] = {0.f, 0.f, 0.f, 0.f};
      const uint32_t a_base = Qs_a + (uint32_t)(16 * hg + (lane & 15)) * kAttPitch + (lane >> 4) * 16;
      const uint32_t b_base = KVs_a + (uint32_t)(buf * kAttTile + 8 * lq + (lane & 7)) * kAttPitch + (lane >> 3) * 16;
#pragma unroll 6
      for (int k0 = 0; k0 < kAttD; k0 += 32) {
        uint32_t a0, a1, a2, a3, c0, c1, c2, c3, b0, b1, b2, b3;
        ldsm_x4(a_base + k0 * 2, a0, a1, a2, a3);
        ldsm_x4(a_base + k0 * 2 + 32, c0, c1, c2, c3);
        ldsm_x4(b_base + k0 * 2, b0, b1, b2, b3);
        mma_bf16_16816(s, a0, a1, a2, a3, b0, b1);
        mma_bf16_16816(s, c0, c1, c2, c3, b2, b3);
      }
      const int tok0 = tile * kAttTile + 8 * lq + 2 * t;
      float2 lo, hi;
      lo.x = tok0 < seq ? s[0] * scale : -INFINITY;
      lo.y = tok0 + 1 < seq ? s[1] * scale : -INFINITY;
      hi.x = tok0 < seq ? s[2] * scale : -INFINITY;
      hi.y = tok0 + 1 < seq ? s[3] * scale : -INFINITY;
      *reinterpret_cast<float2 *>(Ss + (16 * hg + g) * kAttSPitch + 8 * lq + 2 * t) = lo;
      *reinterpret_cast<float2 *>(Ss + (16 * hg + g + 8) * kAttSPitch + 8 * lq + 2 * t) = hi;
    }
    __syncthreads();

    // ---- online softmax for rows g and g+8 of head group hg (every latent quarter repeats it) ----
    uint32_t pa[2][4];
    {
      const float *r_lo = Ss + (16 * hg + g) * kAttSPitch + 2 * t;
      const float *r_hi = r_lo + 8 * kAttSPitch;
      float2 v_lo[4], v_hi[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        v_lo[i] = *reinterpret_cast<const float2 *>(r_lo + 8 * i);
        v_hi[i] = *reinterpret_cast<const float2 *>(r_hi + 8 * i);
      }
      float mx_lo = -INFINITY, mx_hi = -INFINITY;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        mx_lo = fmaxf(mx_lo, fmaxf(v_lo[i].x, v_lo[i].y));
        mx_hi = fmaxf(mx_hi, fmaxf(v_hi[i].x, v_hi[i].y));
      }
      mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 1));
      mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 2));
      mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 1));
      mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 2));
      const float mn_lo = fmaxf(m_lo, mx_lo), mn_hi = fmaxf(m_hi, mx_hi);
      const float mu_lo = mn_lo == -INFINITY ? 0.f : mn_lo, mu_hi = mn_hi == -INFINITY ? 0.f : mn_hi;
      const float al_lo = expf(m_lo - mu_lo), al_hi = expf(m_hi - mu_hi);
      m_lo = mn_lo;
      m_hi = mn_hi;
      float sum_lo = 0.f, sum_hi = 0.f;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        // the probabilities enter the second product rounded to bf16 (as the reference rounds them, :466);
        // the normaliser sums the same rounded values
        float p0 = round_bf16(expf(v_lo[i].x - mu_lo)), p1 = round_bf16(expf(v_lo[i].y - mu_lo));
        float p2 = round_bf16(expf(v_hi[i].x - mu_hi)), p3 = round_bf16(expf(v_hi[i].y - mu_hi));
        sum_lo += p0 + p1;
        sum_hi += p2 + p3;
        // tokens 8i+2t, 8i+2t+1: k-step i/2, low (i even) or high (i odd) half of the k index
        pa[i >> 1][(i & 1) * 2 + 0] = pack_bf16x2(p0, p1);
        pa[i >> 1][(i & 1) * 2 + 1] = pack_bf16x2(p2, p3);
      }
      sum_lo += __shfl_xor_sync(0xffffffffu, sum_lo, 1);
      sum_lo += __shfl_xor_sync(0xffffffffu, sum_lo, 2);
      sum_hi += __shfl_xor_sync(0xffffffffu, sum_hi, 1);
      sum_hi += __shfl_xor_sync(0xffffffffu, sum_hi, 2);
      l_lo = l_lo * al_lo + sum_lo;
      l_hi = l_hi * al_hi + sum_hi;
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        o[j][0] *= al_lo;
        o[j][1] *= al_lo;
        o[j][2] *= al_hi;
        o[j][3] *= al_hi;
      }
    }

    // ---- O += P . C for latent columns [128lq, +128) ---------------------------------------------
    {
      const uint32_t v_base = KVs_a + (uint32_t)(buf * kAttTile + (lane & 15)) * kAttPitch + (128 * lq + (lane >> 4) * 8) * 2;
#pragma unroll
      for (int ks = 0; ks < 2; ++ks) {
#pragma unroll
        for (int jp = 0; jp < 8; ++jp) {
          uint32_t r0, r1, r2, r3;
          ldsm_x4_trans(v_base + (uint32_t)(ks * 16) * kAttPitch + jp * 32, r0, r1, r2, r3);
          mma_bf16_16816(o[2 * jp], pa[ks][0], pa[ks][1], pa[ks][2], pa[ks][3], r0, r1);
          mma_bf16_16816(o[2 * jp + 1], pa[ks][0], pa[ks][1], pa[ks][2], pa[ks][3], r2, r3);
        }
      }
    }
    __syncthreads();  // the tile buffer and the score tile are free again
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");

  float *po = part_o + ((size_t)b * splits + split) * kAttHeads * kAttDV;
#pragma unroll
  for (int j = 0; j < 16; ++j) {
    const int col = 128 * lq + 8 * j + 2 * t;
    *reinterpret_cast<float2 *>(po + (size_t)(16 * hg + g) * kAttDV + col) = make_float2(o[j][0], o[j][1]);
    *reinterpret_cast<float2 *>(po + (size_t)(16 * hg + g + 8) * kAttDV + col) = make_float2(o[j][2], o[j][3]);
  }
  if (lq == 0 && t == 0) {
    my_ml[(16 * hg + g) * 2] = m_lo;
    my_ml[(16 * hg + g) * 2 + 1] = l_lo;
    my_ml[(16 * hg + g + 8) * 2] = m_hi;
    my_ml[(16 * hg + g + 8) * 2 + 1] = l_hi;
  }
}

int launch_mla_attend(const uint16_t *q, const uint16_t *cache, long ctx_stride, const int *seq_len, int B, int splits,
                      float scale, float *part_o, float *part_ml, cudaStream_t stream) {
  static bool configured = false;
  const size_t smem = mla_attend_smem_bytes();
  if (!configured) {
    BLOK_CUDA(cudaFuncSetAttribute(mla_attend_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    configured = true;
  }
  mla_attend_kernel<false><<<dim3(splits, B), kAttThreads, smem, stream>>>(q, cache, ctx_stride, seq_len, scale, part_o,
                                                                          part_ml, nullptr, nullptr, 0, 0);
  return launch_status("mla_attend_kernel");
}

// The same over a paged pool: page_rows must be a positive multiple of the kernel's 32-row tile.
int launch_mla_attend_paged(const uint16_t *q, const uint16_t *pool, const int *block_table, const int *slot_of,
                            int table_stride, int page_rows, const int *seq_len, int B, int splits, float scale,
                            float *part_o, float *part_ml, cudaStream_t stream) {
  static bool configured = false;
  const size_t smem = mla_attend_smem_bytes();
  if (!configured) {
    BLOK_CUDA(cudaFuncSetAttribute(mla_attend_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    configured = true;
  }
  mla_attend_kernel<true><<<dim3(splits, B), kAttThreads, smem, stream>>>(q, pool, 0, seq_len, scale, part_o, part_ml,
                                                                         block_table, slot_of, table_stride, page_rows);
  return launch_status("mla_attend_kernel(paged)");
}

}  // namespace blok
