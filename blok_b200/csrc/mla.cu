// MLA decode attention in the absorbed form over a bf16 latent cache.
// Reference: src/kimi_exec.cu:813-826 (projections, RMSNorm, RoPE, KV store, o_proj)
// and :692-716 / :414-475 (three-pass softmax attention over materialised K/V).
//
// The reference stores, per token and layer, the full K [64 x 192] and V [64 x 128]
// in fp32 (81,920 B) and re-reads K three times.  Both are functions of the bf16
// latent row (normed c_kv [512], roped k_pe [64]) that the reference computes at
// :817-823, so the cache here is that row, 1,152 B per token, and the attention is
// evaluated in the latent space:
//   q_abs_h = W_UK_h^T q_nope_h        W_UK_h = kv_b rows [h*256, h*256+128)   (:366-369)
//   s_t     = (q_abs_h . c_t + q_rope_h . kpe_t) * scale
//   o_lat_h = sum_t softmax(s)_t c_t
//   out_h   = W_UV_h o_lat_h           W_UV_h = kv_b rows [h*256+128, h*256+256)
// One pass over the cache with an online softmax; the sequence is split over CTAs
// (flash-decoding) and the partial results are merged by a second kernel.
#include <cmath>
#include <cstdlib>
#include <cstring>
#include <new>

#include "bf16_mma.cuh"
#include "wgemm.h"

namespace blok {

int launch_bf16_gemv(const uint16_t *w, const uint16_t *x, uint16_t *y_bf16, float *y_f32, int rows, int cols, int T,
                     cudaStream_t stream);
size_t bf16_gemv_splitk_workspace_bytes(int rows);
int launch_bf16_gemv_splitk_pair(const uint16_t *w1, int rows1, uint16_t *y1, const uint16_t *w2, int rows2, uint16_t *y2,
                                 const uint16_t *x, int cols, int T, void *ws, size_t ws_bytes, cudaStream_t stream);
int launch_bf16_gemv_splitk(const uint16_t *w, const uint16_t *x, uint16_t *y_bf16, float *y_f32, int rows, int cols, int T,
                            void *ws, size_t ws_bytes, cudaStream_t stream);

// ---------------------------------------------------------------------------
// Per-head mat-vec for up to 8 tokens: y[tok, head, r] = sum_c W[head][r][c] * x[tok, head, c].
// grid = (rows/16, heads), 4 warps split K.  Strides are in elements.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(128)
    bf16_head_gemv_kernel(const uint16_t *__restrict__ w, long w_head_stride, const uint16_t *__restrict__ x,
                          long x_tok_stride, long x_head_stride, uint16_t *__restrict__ y, long y_tok_stride,
                          long y_head_stride, int cols, int T_all) {
  extern __shared__ __align__(16) unsigned char smem[];
  __shared__ float partial[4][16][8];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int head = blockIdx.y;
  // blockIdx.z: the group of 8 tokens (the later groups find the head's matrix in L2)
  const int T = min(8, T_all - 8 * (int)blockIdx.z);
  x += (size_t)blockIdx.z * 8 * x_tok_stride;
  y += (size_t)blockIdx.z * 8 * y_tok_stride;
  const int per_row = cols / 8;
  for (int u = tid; u < per_row * T; u += blockDim.x) {
    int tok = u / per_row, c = u - tok * per_row;
    uint4 v = reinterpret_cast<const uint4 *>(x + (size_t)tok * x_tok_stride + (size_t)head * x_head_stride)[c];
    reinterpret_cast<uint4 *>(smem + tok * bf16_x_row_bytes(cols))[c] = v;
  }
  __syncthreads();
  const size_t wrow = cols / 8;
  const int row0 = blockIdx.x * 16;
  const uint4 *w_lo = reinterpret_cast<const uint4 *>(w + (size_t)head * w_head_stride) + (size_t)(row0 + g) * wrow;
  const uint4 *w_hi = w_lo + 8 * wrow;
  const int tok = g < T ? g : T - 1;
  const uint4 *xrow = reinterpret_cast<const uint4 *>(smem + tok * bf16_x_row_bytes(cols)) + t;
  const int ksteps = cols / 32;
  const int base = ksteps / 4, rem = ksteps % 4;
  const int ks0 = warp * base + (warp < rem ? warp : rem);
  const int nsteps = base + (warp < rem ? 1 : 0);
  float d[4] = {0.f, 0.f, 0.f, 0.f};
  bf16_rows16_accumulate(w_lo, w_hi, xrow, ks0, nsteps, t, d);
  partial[warp][g][2 * t] = d[0];
  partial[warp][g][2 * t + 1] = d[1];
  partial[warp][g + 8][2 * t] = d[2];
  partial[warp][g + 8][2 * t + 1] = d[3];
  __syncthreads();
  if (tid < 128) {
    int r = tid >> 3, tk = tid & 7;
    if (tk < T) {
      float v = partial[0][r][tk] + partial[1][r][tk] + partial[2][r][tk] + partial[3][r][tk];
      y[(size_t)tk * y_tok_stride + (size_t)head * y_head_stride + row0 + r] = f32_to_bf16_bits(v);
    }
  }
}

// ---------------------------------------------------------------------------
// Per sequence: RMSNorm of c_kv, RoPE of k_pe, append to the cache; RoPE of the
// query's rope part into q_full.  src/kimi_exec.cu:817 (norm), :346-357 (rope).
//   kva    bf16 [B, kv_rank + rope]   output of kv_a_proj_with_mqa
//   q      bf16 [B, heads, nope + rope]
//   q_full bf16 [B, heads, kv_rank + rope]; this kernel writes columns [kv_rank, kv_rank+rope)
// ---------------------------------------------------------------------------
// grid = (1 + heads / 8, B), 256 threads: block 0 of a sequence normalises c_kv, rotates k_pe, appends the cache row
// and publishes seq = ctx_len + 1 (the tokens the attention covers); blocks 1.. rotate the rope part of 8 heads each.
__global__ void __launch_bounds__(256) mla_prep_kernel(const uint16_t *__restrict__ kva, const uint16_t *__restrict__ kva_ln,
                                                       const uint16_t *__restrict__ q, const float *__restrict__ inv_freq,
                                                       const int *__restrict__ ctx_len, uint16_t *__restrict__ cache,
                                                       long ctx_stride, uint16_t *__restrict__ q_full, int *__restrict__ seq,
                                                       int heads, int nope, int rope, int kv_rank, float eps,
                                                       const int *__restrict__ block_table, const int *__restrict__ slot_of,
                                                       int table_stride, int page_rows, long ctx_cap, unsigned *__restrict__ err) {
  __shared__ float red[32];
  const int b = blockIdx.y, tid = threadIdx.x;
  int pos = ctx_len[b];
  // A position outside the sequence's rows (dense: ctx_cap rows; paged: table_stride pages) must not become a store or
  // a read: the row is not written, the attention is kept inside the rows, and the host learns of it from *err.
  const bool in_range = pos >= 0 && (long)pos < ctx_cap;
  if (!in_range) pos = pos < 0 ? 0 : (int)(ctx_cap - 1);
  const int half = rope / 2, lat_w = kv_rank + rope;
  if (blockIdx.x > 0) {
    // thread = (head, pair): interleaved pair (2p, 2p+1) -> de-interleaved (p, half+p); every product rounded (:353-356)
    const int i = (blockIdx.x - 1) * 256 + tid;
    if (i < heads * half) {
      const int h = i / half, p = i - h * half;
      const float ang = pos * inv_freq[p];
      const float c = round_bf16(cosf(ang)), s = round_bf16(sinf(ang));
      const uint16_t *qr = q + ((size_t)b * heads + h) * (nope + rope) + nope;
      uint16_t *qo = q_full + ((size_t)b * heads + h) * lat_w + kv_rank;
      const uint32_t pair = *reinterpret_cast<const uint32_t *>(qr + 2 * p);
      const float x0 = bf16lo(pair), x1 = bf16hi(pair);
      qo[p] = f32_to_bf16_bits(round_bf16(x0 * c) - round_bf16(x1 * s));
      qo[half + p] = f32_to_bf16_bits(round_bf16(x1 * c) + round_bf16(x0 * s));
    }
    return;
  }
  if (tid == 0) {
    seq[b] = pos + 1;
    if (!in_range) atomicExch(err, 1u + (unsigned)b);
  }
  if (!in_range) return;
  const uint16_t *kr = kva + (size_t)b * lat_w;
  // dense: sequence b's rows start at b * ctx_stride; paged: the row's page comes from the sequence's block table
  uint16_t *row = block_table
                      ? cache + ((size_t)block_table[(size_t)(slot_of ? slot_of[b] : b) * table_stride + pos / page_rows] * page_rows +
                                 pos % page_rows) * lat_w
                      : cache + ((size_t)b * ctx_stride + pos) * lat_w;
  float v = 0.f;
  for (int i = tid; i < kv_rank; i += blockDim.x) {
    float a = bf16_bits_to_f32(kr[i]);
    v = fmaf(a, a, v);
  }
  v = warp_sum(v);
  if ((tid & 31) == 0) red[tid >> 5] = v;
  __syncthreads();
  if (tid < 32) {
    float s = tid < (blockDim.x >> 5) ? red[tid] : 0.f;
    s = warp_sum(s);
    if (tid == 0) red[0] = s;
  }
  __syncthreads();
  const float scale = rsqrtf(red[0] / kv_rank + eps);
  for (int i = tid; i < kv_rank; i += blockDim.x)
    row[i] = f32_to_bf16_bits(round_bf16(bf16_bits_to_f32(kr[i]) * scale) * bf16_bits_to_f32(kva_ln[i]));
  if (tid < half) {
    const int p = tid;
    const float ang = pos * inv_freq[p];
    const float c = round_bf16(cosf(ang)), s = round_bf16(sinf(ang));
    const float x0 = bf16_bits_to_f32(kr[kv_rank + 2 * p]), x1 = bf16_bits_to_f32(kr[kv_rank + 2 * p + 1]);
    row[kv_rank + p] = f32_to_bf16_bits(round_bf16(x0 * c) - round_bf16(x1 * s));
    row[kv_rank + half + p] = f32_to_bf16_bits(round_bf16(x1 * c) + round_bf16(x0 * s));
  }
}

// ctx[i] = first[0] + i: the positions of the T consecutive tokens of a prefill chunk.
__global__ void mla_chunk_positions_kernel(const int *__restrict__ first, int T, int *__restrict__ ctx) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < T) ctx[i] = first[0] + i;
}

// W_UK^T: out[h][j][d] = kv_b[h*(nope+v) + d][j]  (a pure re-arrangement, no arithmetic)
__global__ void transpose_wuk_kernel(const uint16_t *__restrict__ kv_b, uint16_t *__restrict__ out, int heads, int nope,
                                     int v_head, int kv_rank) {
  long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
  long total = (long)heads * kv_rank * nope;
  if (i >= total) return;
  int d = (int)(i % nope);
  long r = i / nope;
  int j = (int)(r % kv_rank);
  int h = (int)(r / kv_rank);
  out[i] = kv_b[((size_t)h * (nope + v_head) + d) * kv_rank + j];
}

// ---------------------------------------------------------------------------
// Merge of the split-KV partial results.  grid = (heads, B), 128 threads.
//   part_o fp32 [B, splits, heads, kv_rank] unnormalised, part_ml fp32 [B, splits, heads, 2] = (max, sum)
// ---------------------------------------------------------------------------
__global__ void mla_merge_kernel(const float *__restrict__ part_o, const float *__restrict__ part_ml, int splits,
                                 int heads, int kv_rank, uint16_t *__restrict__ o_lat) {
  extern __shared__ float s_wt[];  // [splits] weight of every split: exp(m_s - M), 0 for an empty split
  __shared__ float s_red[2][4];
  const int h = blockIdx.x, b = blockIdx.y, tid = threadIdx.x;
  const float *ml = part_ml + ((size_t)b * splits * heads + h) * 2;  // split s at + s * heads * 2
  float M = -INFINITY;
  for (int s = tid; s < splits; s += blockDim.x) M = fmaxf(M, ml[(size_t)s * heads * 2]);
  M = warp_max(M);
  if ((tid & 31) == 0) s_red[0][tid >> 5] = M;
  __syncthreads();
  M = fmaxf(fmaxf(s_red[0][0], s_red[0][1]), fmaxf(s_red[0][2], s_red[0][3]));
  float L = 0.f;
  for (int s = tid; s < splits; s += blockDim.x) {
    const float m = ml[(size_t)s * heads * 2];
    const float wt = m != -INFINITY ? expf(m - M) : 0.f;
    s_wt[s] = wt;
    L += wt * ml[(size_t)s * heads * 2 + 1];
  }
  L = warp_sum(L);
  if ((tid & 31) == 0) s_red[1][tid >> 5] = L;
  __syncthreads();
  L = (s_red[1][0] + s_red[1][1]) + (s_red[1][2] + s_red[1][3]);
  const float inv = L > 0.f ? 1.0f / L : 0.f;
  const float *po = part_o + ((size_t)b * splits * heads + h) * kv_rank;  // split s at + s * heads * kv_rank
  // four columns per thread, eight splits' worth of loads in flight per thread: the partial results (B x splits x 128 KB)
  // come from L2 or HBM, and the kernel is as fast as it keeps bytes in flight.  Each column still adds its splits in
  // ascending order.
  const float4 *po4 = reinterpret_cast<const float4 *>(po);
  const size_t stride4 = (size_t)heads * kv_rank / 4;
  for (int j4 = tid; j4 < kv_rank / 4; j4 += blockDim.x) {
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    int s = 0;
    for (; s + 8 <= splits; s += 8) {
      float4 v[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) v[i] = __ldg(po4 + (size_t)(s + i) * stride4 + j4);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float wt = s_wt[s + i];
        acc.x = fmaf(wt, v[i].x, acc.x);
        acc.y = fmaf(wt, v[i].y, acc.y);
        acc.z = fmaf(wt, v[i].z, acc.z);
        acc.w = fmaf(wt, v[i].w, acc.w);
      }
    }
    for (; s < splits; ++s) {
      const float4 v = __ldg(po4 + (size_t)s * stride4 + j4);
      const float wt = s_wt[s];
      acc.x = fmaf(wt, v.x, acc.x);
      acc.y = fmaf(wt, v.y, acc.y);
      acc.z = fmaf(wt, v.z, acc.z);
      acc.w = fmaf(wt, v.w, acc.w);
    }
    uint2 o;
    o.x = pack_bf16x2(acc.x * inv, acc.y * inv);
    o.y = pack_bf16x2(acc.z * inv, acc.w * inv);
    *reinterpret_cast<uint2 *>(o_lat + ((size_t)b * heads + h) * kv_rank + (size_t)j4 * 4) = o;
  }
}

size_t mla_attend_smem_bytes();
int launch_mla_attend(const uint16_t *q, const uint16_t *cache, long ctx_stride, const int *seq_len, int B, int splits,
                      float scale, float *part_o, float *part_ml, cudaStream_t stream);
int launch_mla_attend_tc(const uint16_t *q, const uint16_t *cache, long ctx_stride, long total_rows, const int *seq_len, int B, int splits,
                         float scale, float *part_o, float *part_ml, cudaStream_t stream);
int launch_mla_attend_tc_paged(const uint16_t *q, const uint16_t *pool, long pool_rows, const int *block_table, const int *slot_of,
                               int table_stride, int page_rows, const int *seq_len, int B, int splits, float scale, float *part_o,
                               float *part_ml, cudaStream_t stream);
int mla_attend_tc_take_error(unsigned *out);
int mla_attend_tc_trace(long long *host_out, int max_entries);
int launch_mla_attend_paged(const uint16_t *q, const uint16_t *pool, const int *block_table, const int *slot_of,
                            int table_stride, int page_rows, const int *seq_len, int B, int splits, float scale,
                            float *part_o, float *part_ml, cudaStream_t stream);

static int launch_head_gemv(const uint16_t *w, long w_head_stride, const uint16_t *x, long x_tok_stride,
                            long x_head_stride, uint16_t *y, long y_tok_stride, long y_head_stride, int rows, int cols,
                            int heads, int T, cudaStream_t stream) {
  size_t smem = bf16_x_row_bytes(cols) * std::min(T, 8);
  bf16_head_gemv_kernel<<<dim3(rows / 16, heads, (T + 7) / 8), 128, smem, stream>>>(w, w_head_stride, x, x_tok_stride, x_head_stride,
                                                                      y, y_tok_stride, y_head_stride, cols, T);
  return launch_status("bf16_head_gemv_kernel");
}

static size_t align256(size_t v) { return (v + 255) / 256 * 256; }

constexpr int kMlaMaxBatch = 64;  // sequences (or tokens of a prefill chunk) per call: what one pass of the weight-streaming kernel covers

}  // namespace blok

struct blok_mla_layer {
  blok_mla_weights w;
  int max_batch = 0;
  int max_splits = 0;
  float scale = 0.f;
  void *ws = nullptr;
  uint16_t *wuk_t = nullptr;   // [heads, kv_rank, qk_nope]
  float *inv_freq = nullptr;   // [qk_rope / 2]
  uint16_t *qa = nullptr;      // [B, q_rank]
  uint16_t *q = nullptr;       // [B, heads, nope + rope]
  uint16_t *kva = nullptr;     // [B, kv_rank + rope]
  uint16_t *q_full = nullptr;  // [B, heads, kv_rank + rope]
  uint16_t *o_lat = nullptr;   // [B, heads, kv_rank]
  uint16_t *av = nullptr;      // [B, heads * v_head]
  int *seq = nullptr;          // [B]
  unsigned *err = nullptr;     // [1] 1 + b when entry b of a call had a position outside its sequence's rows
  int *chunk_pos = nullptr;    // [B] positions of a prefill chunk's tokens
  int *tiles = nullptr;        // tile table of the weight-streaming GEMM (projections of 16 or more entries)
  int n_tiles = 0;
  void *sk_ws = nullptr;       // split-K partial sums and tickets of the projections (zeroed at create)
  size_t sk_bytes = 0;
  float *wg_ws = nullptr;      // K-split partial sums of the projections over 9..64 entries (wgemm_stream.cu)
  size_t wg_bytes = 0;
  float *part_o = nullptr;     // [max_splits * max_batch..]
  float *part_ml = nullptr;
};

using namespace blok;

// YaRN inverse frequencies, src/kimi_exec.cu:325-344 with the factor as a parameter.
static void yarn_inv_freq_host(const blok_mla_weights &w, float *out) {
  const float dim = (float)w.qk_rope;
  auto corr = [&](float rotations) {
    return dim * logf(w.yarn_original_ctx / (rotations * 2.0f * 3.141592654f)) / (2.0f * logf(w.rope_theta));
  };
  float low = fmaxf(floorf(corr(w.yarn_beta_fast)), 0.0f);
  float high = fminf(ceilf(corr(w.yarn_beta_slow)), dim - 1.0f);
  if (low == high) high += 0.001f;
  for (int p = 0; p < w.qk_rope / 2; ++p) {
    float extra = powf(w.rope_theta, -2.0f * (float)p / dim);
    float inter = extra / w.yarn_factor;
    float ramp = fminf(1.0f, fmaxf(0.0f, ((float)p - low) / (high - low)));
    float mask = 1.0f - ramp;
    out[p] = inter * (1.0f - mask) + extra * mask;
  }
}

extern "C" float blok_mla_softmax_scale(const blok_mla_weights *w) {
  if (!w) return 0.f;
  float mscale = 0.1f * w->yarn_mscale_all_dim * logf(w->yarn_factor) + 1.0f;
  return (1.0f / sqrtf((float)(w->qk_nope + w->qk_rope))) * mscale * mscale;
}

extern "C" int blok_mla_layer_create(const blok_mla_weights *w, int max_batch, int max_ctx, blok_mla_layer_t **out) {
  BLOK_REQUIRE(w && out, BLOK_ERR_ARG, "blok_mla_layer_create: null pointer");
  BLOK_REQUIRE(max_batch >= 1 && max_batch <= kMlaMaxBatch && max_ctx >= 1, BLOK_ERR_ARG,
               "blok_mla_layer_create: need 1 <= max_batch <= %d and max_ctx >= 1", kMlaMaxBatch);
  BLOK_REQUIRE(w->heads == 64 && w->kv_rank == 512 && w->qk_rope == 64 && w->qk_nope % 32 == 0 && w->v_head % 16 == 0 &&
                   w->hidden % 32 == 0 && w->q_rank % 32 == 0,
               BLOK_ERR_SHAPE,
               "blok_mla_layer_create: the attention kernel is built for 64 heads, kv_rank 512, qk_rope 64 (got %d, %d, %d)",
               w->heads, w->kv_rank, w->qk_rope);
  BLOK_REQUIRE(w->q_a && w->q_a_ln && w->q_b && w->kv_a && w->kv_a_ln && w->kv_b && w->o, BLOK_ERR_ARG,
               "blok_mla_layer_create: weight pointer missing");
  BLOK_REQUIRE(w->yarn_factor > 0.f && w->rope_theta > 1.f, BLOK_ERR_ARG, "blok_mla_layer_create: bad rope parameters");
  blok_mla_layer *L = new (std::nothrow) blok_mla_layer();
  BLOK_REQUIRE(L, BLOK_ERR_ARG, "blok_mla_layer_create: out of host memory");
  L->w = *w;
  L->max_batch = max_batch;
  L->max_splits = sm_count();
  L->scale = blok_mla_softmax_scale(w);
  const int lat_w = w->kv_rank + w->qk_rope, qk_head = w->qk_nope + w->qk_rope;
  size_t off = 0;
  auto take = [&](size_t bytes) {
    size_t at = off;
    off = align256(off + bytes);
    return at;
  };
  size_t o_wuk = take((size_t)w->heads * w->kv_rank * w->qk_nope * 2);
  size_t o_freq = take((size_t)(w->qk_rope / 2) * 4);
  size_t o_qa = take((size_t)max_batch * w->q_rank * 2);
  size_t o_q = take((size_t)max_batch * w->heads * qk_head * 2);
  size_t o_kva = take((size_t)max_batch * lat_w * 2);
  size_t o_qf = take((size_t)max_batch * w->heads * lat_w * 2);
  size_t o_ol = take((size_t)max_batch * w->heads * w->kv_rank * 2);
  size_t o_av = take((size_t)max_batch * w->heads * w->v_head * 2);
  size_t o_seq = take((size_t)max_batch * 4);
  size_t o_cpos = take((size_t)max_batch * 4);
  size_t o_err = take(4);
  L->n_tiles = (max_batch + kWgTileTokens - 1) / kWgTileTokens;
  size_t o_tiles = take((size_t)(3 * L->n_tiles + 1) * sizeof(int));
  size_t o_po = take((size_t)(L->max_splits + max_batch) * w->heads * w->kv_rank * 4);
  size_t o_pml = take((size_t)(L->max_splits + max_batch) * w->heads * 2 * 4);
  L->sk_bytes = bf16_gemv_splitk_workspace_bytes(std::max(std::max(w->q_rank, lat_w), std::max(w->heads * qk_head, w->hidden)));
  size_t o_sk = take(L->sk_bytes);
  if (max_batch > 8) {
    const int mb = std::min(max_batch, kWgStreamTokens);
    L->wg_bytes = std::max(std::max(wgemm_splitk_bytes(WG_BF16_PLAIN, w->hidden, w->q_rank, mb), wgemm_splitk_bytes(WG_BF16_PLAIN, w->hidden, lat_w, mb)),
                           std::max(wgemm_splitk_bytes(WG_BF16_PLAIN, w->q_rank, w->heads * qk_head, mb),
                                    wgemm_splitk_bytes(WG_BF16_PLAIN, w->heads * w->v_head, w->hidden, mb)));
  }
  size_t o_wg = take(std::max(L->wg_bytes, (size_t)16));
  cudaError_t e = cudaMalloc(&L->ws, off);
  if (e != cudaSuccess) {
    delete L;
    return cuda_fail(e, "cudaMalloc(mla layer workspace)");
  }
  e = cudaMemset(L->ws, 0, off);  // the split-K tickets start at zero
  if (e != cudaSuccess) {
    cudaFree(L->ws);
    delete L;
    return cuda_fail(e, "cudaMemset(mla layer workspace)");
  }
  unsigned char *b = static_cast<unsigned char *>(L->ws);
  L->wuk_t = reinterpret_cast<uint16_t *>(b + o_wuk);
  L->inv_freq = reinterpret_cast<float *>(b + o_freq);
  L->qa = reinterpret_cast<uint16_t *>(b + o_qa);
  L->q = reinterpret_cast<uint16_t *>(b + o_q);
  L->kva = reinterpret_cast<uint16_t *>(b + o_kva);
  L->q_full = reinterpret_cast<uint16_t *>(b + o_qf);
  L->o_lat = reinterpret_cast<uint16_t *>(b + o_ol);
  L->av = reinterpret_cast<uint16_t *>(b + o_av);
  L->seq = reinterpret_cast<int *>(b + o_seq);
  L->chunk_pos = reinterpret_cast<int *>(b + o_cpos);
  L->err = reinterpret_cast<unsigned *>(b + o_err);
  L->tiles = reinterpret_cast<int *>(b + o_tiles);
  L->part_o = reinterpret_cast<float *>(b + o_po);
  L->part_ml = reinterpret_cast<float *>(b + o_pml);
  L->sk_ws = b + o_sk;
  L->wg_ws = reinterpret_cast<float *>(b + o_wg);
  float freq[128];
  yarn_inv_freq_host(*w, freq);
  e = cudaMemcpy(L->inv_freq, freq, (size_t)(w->qk_rope / 2) * 4, cudaMemcpyHostToDevice);
  if (e == cudaSuccess) {
    long total = (long)w->heads * w->kv_rank * w->qk_nope;
    transpose_wuk_kernel<<<(unsigned)((total + 255) / 256), 256>>>(w->kv_b, L->wuk_t, w->heads, w->qk_nope, w->v_head,
                                                                   w->kv_rank);
    count_launch();
    e = cudaDeviceSynchronize();
  }
  if (e != cudaSuccess) {
    cudaFree(L->ws);
    delete L;
    return cuda_fail(e, "blok_mla_layer_create: set-up");
  }
  (void)max_ctx;
  *out = L;
  return BLOK_OK;
}

extern "C" int blok_mla_layer_refresh(blok_mla_layer_t *L) {
  BLOK_REQUIRE(L, BLOK_ERR_ARG, "blok_mla_layer_refresh: null pointer");
  const blok_mla_weights &w = L->w;
  const long total = (long)w.heads * w.kv_rank * w.qk_nope;
  transpose_wuk_kernel<<<(unsigned)((total + 255) / 256), 256>>>(w.kv_b, L->wuk_t, w.heads, w.qk_nope, w.v_head, w.kv_rank);
  count_launch();
  BLOK_CUDA(cudaDeviceSynchronize());
  return launch_status("transpose_wuk_kernel");
}

extern "C" int blok_mla_layer_destroy(blok_mla_layer_t *L) {
  if (!L) return BLOK_OK;
  cudaError_t e = L->ws ? cudaFree(L->ws) : cudaSuccess;
  delete L;
  return e == cudaSuccess ? BLOK_OK : cuda_fail(e, "cudaFree(mla layer workspace)");
}

extern "C" int blok_mla_attend_trace(long long *host_out, int max_entries) {
  if (!host_out || max_entries <= 0) return 0;
  return mla_attend_tc_trace(host_out, max_entries);
}

extern "C" int blok_mla_layer_check(blok_mla_layer_t *L, blok_stream_t stream) {
  BLOK_REQUIRE(L, BLOK_ERR_ARG, "blok_mla_layer_check: null pointer");
  BLOK_CUDA(cudaStreamSynchronize((cudaStream_t)stream));
  unsigned tc_err = 0;
  if (int rc = mla_attend_tc_take_error(&tc_err)) return rc;
  if (tc_err) {
    set_error("blok_mla_decode: the attention core gave up on wait %u (1 tile buffer, 2-5 MMA thread, 6-9 softmax warps)", tc_err);
    return BLOK_ERR_TIMEOUT;
  }
  unsigned err = 0;
  BLOK_CUDA(cudaMemcpy(&err, L->err, sizeof(err), cudaMemcpyDeviceToHost));
  if (err == 0) return BLOK_OK;
  BLOK_CUDA(cudaMemset(L->err, 0, sizeof(err)));
  set_error("blok_mla_decode: entry %u had a position outside its sequence's cache rows; its row was not stored", err - 1);
  return BLOK_ERR_SHAPE;
}

// Where the latent rows of the sequences of a call live.
struct CacheRef {
  uint16_t *base = nullptr;         // dense cache, or the page pool
  long seq_stride = 0;              // dense: rows between consecutive sequences; 0 = every entry is the same sequence
  long ctx_cap = 0;                 // rows one sequence can hold (bounds the context splits)
  const int *block_table = nullptr; // paged when non-null: int32 [slots, table_stride] page numbers
  const int *slot_of = nullptr;     // paged: table row of batch entry b (null: b)
  int table_stride = 0, page_rows = 0;
};

// Context splits per sequence: enough CTAs to fill the GPU, but never more than one per 64 rows of the cache
// allocation (the sequence lengths live on the device; the capacity bounds them), so that a short cache is not cut
// into slivers whose merge costs more than the attention.
static int splits_for(const blok_mla_layer *L, int B, long ctx_cap) {
  long s = L->max_splits / B;
  const long cap = (ctx_cap + 63) / 64;
  if (s > cap) s = cap;
  return s < 1 ? 1 : (int)s;
}

static int attend_and_merge(blok_mla_layer *L, const uint16_t *q, const CacheRef &c, const int *seq_len, int B, float scale,
                            uint16_t *o_lat, cudaStream_t stream) {
  const int splits = splits_for(L, B, c.ctx_cap);
  // the tcgen05 core by default; BLOK_MLA_ATTEND_IMPL=mma (read at every call) selects the mma.sync kernel, which also
  // serves page sizes that are not a multiple of the tcgen05 core's 64-token tile
  const char *impl = getenv("BLOK_MLA_ATTEND_IMPL");
  const bool tc = !(impl && strcmp(impl, "mma") == 0) && (!c.block_table || c.page_rows % 64 == 0);
  int rc;
  if (tc) {
    // the rows the tensor map may address: the whole dense cache (reads past it give zeros); a paged tile never leaves
    // its page, so the pool needs no tighter bound than the coordinate range
    const long dense_rows = c.seq_stride > 0 ? (long)B * c.seq_stride : c.ctx_cap;
    rc = c.block_table ? launch_mla_attend_tc_paged(q, c.base, (1l << 31) - 64, c.block_table, c.slot_of, c.table_stride, c.page_rows, seq_len,
                                                    B, splits, scale, L->part_o, L->part_ml, stream)
                       : launch_mla_attend_tc(q, c.base, c.seq_stride, dense_rows, seq_len, B, splits, scale, L->part_o, L->part_ml, stream);
  } else
    rc = c.block_table ? launch_mla_attend_paged(q, c.base, c.block_table, c.slot_of, c.table_stride, c.page_rows, seq_len, B,
                                                 splits, scale, L->part_o, L->part_ml, stream)
                       : launch_mla_attend(q, c.base, c.seq_stride, seq_len, B, splits, scale, L->part_o, L->part_ml, stream);
  if (rc) return rc;
  mla_merge_kernel<<<dim3(L->w.heads, B), 128, (size_t)splits * sizeof(float), stream>>>(L->part_o, L->part_ml, splits, L->w.heads, L->w.kv_rank,
                                                           o_lat);
  return launch_status("mla_merge_kernel");
}

static int check_paged(const char *who, const void *pool, const int *block_table, int table_stride, int page_rows) {
  BLOK_REQUIRE(pool && block_table, BLOK_ERR_ARG, "%s: null pointer", who);
  BLOK_REQUIRE((reinterpret_cast<uintptr_t>(pool) & 15) == 0, BLOK_ERR_ARG, "%s: the pool must be 16-byte aligned", who);
  BLOK_REQUIRE(table_stride >= 1 && page_rows >= 32 && page_rows % 32 == 0, BLOK_ERR_SHAPE,
               "%s: page_rows (%d) must be a positive multiple of 32 and table_stride (%d) >= 1", who, page_rows, table_stride);
  return BLOK_OK;
}

extern "C" int blok_mla_attend(blok_mla_layer_t *L, const blok_bf16_t *q, const blok_bf16_t *cache, long ctx_stride,
                               const int *seq_len, int B, float softmax_scale, blok_bf16_t *o_lat,
                               blok_stream_t stream) {
  BLOK_REQUIRE(L && q && cache && seq_len && o_lat, BLOK_ERR_ARG, "blok_mla_attend: null pointer");
  BLOK_REQUIRE(B >= 1 && B <= L->max_batch && ctx_stride >= 1, BLOK_ERR_SHAPE, "blok_mla_attend: B=%d outside [1, %d]", B,
               L->max_batch);
  BLOK_REQUIRE((reinterpret_cast<uintptr_t>(q) & 15) == 0 && (reinterpret_cast<uintptr_t>(cache) & 15) == 0, BLOK_ERR_ARG,
               "blok_mla_attend: q and cache must be 16-byte aligned");
  CacheRef c;
  c.base = const_cast<uint16_t *>(cache);
  c.seq_stride = c.ctx_cap = ctx_stride;
  return attend_and_merge(L, q, c, seq_len, B, softmax_scale, o_lat, (cudaStream_t)stream);
}

extern "C" int blok_mla_attend_paged(blok_mla_layer_t *L, const blok_bf16_t *q, const blok_bf16_t *pool, const int *block_table,
                                     const int *slot_of, int table_stride, int page_rows, const int *seq_len, int B,
                                     float softmax_scale, blok_bf16_t *o_lat, blok_stream_t stream) {
  BLOK_REQUIRE(L && q && seq_len && o_lat, BLOK_ERR_ARG, "blok_mla_attend_paged: null pointer");
  BLOK_REQUIRE(B >= 1 && B <= L->max_batch, BLOK_ERR_SHAPE, "blok_mla_attend_paged: B=%d outside [1, %d]", B, L->max_batch);
  BLOK_REQUIRE((reinterpret_cast<uintptr_t>(q) & 15) == 0, BLOK_ERR_ARG, "blok_mla_attend_paged: q must be 16-byte aligned");
  if (int rc = check_paged("blok_mla_attend_paged", pool, block_table, table_stride, page_rows)) return rc;
  CacheRef c;
  c.base = const_cast<uint16_t *>(pool);
  c.ctx_cap = (long)table_stride * page_rows;
  c.block_table = block_table;
  c.slot_of = slot_of;
  c.table_stride = table_stride;
  c.page_rows = page_rows;
  return attend_and_merge(L, q, c, seq_len, B, softmax_scale, o_lat, (cudaStream_t)stream);
}

// y[b, :] = bf16(W x[b, :]) for B entries.  Up to 8 entries go through the split-K mat-vec kernel; 9 to 64 through the
// weight-streaming kernel, one pass over the weights for all entries; more, where the matrix fits its tiling, through the
// GEMM (`tiles_ready`: the identity tile table for B entries has been written on this stream), else 8 at a time.
static int project(blok_mla_layer *L, const uint16_t *w, const uint16_t *x, uint16_t *y, int rows, int cols, int B, bool tiles_ready,
                   cudaStream_t stream) {
  if (B > 8 && B <= kWgStreamTokens && rows % 16 == 0 && cols % 256 == 0)
    return launch_wgemm_rows(WG_BF16_PLAIN, w, nullptr, x, y, nullptr, rows, cols, B, L->wg_ws, L->wg_bytes, stream);
  if (tiles_ready && rows % 128 == 0 && cols % 512 == 0) {
    const int tiles = (B + kWgTileTokens - 1) / kWgTileTokens;
    int *tab = L->tiles;
    WgArgs r;
    r.w_a = w; r.w_b = nullptr; r.s_a = r.s_b = nullptr; r.expert_stride_rows = 0; r.x = x; r.x_index = nullptr;
    r.K = cols; r.R = rows; r.out_bf16 = y; r.out_f32 = nullptr;
    r.tile_expert = tab; r.tile_start = tab + L->n_tiles; r.tile_count = tab + 2 * L->n_tiles; r.num_tiles = tab + 3 * L->n_tiles;
    r.out_index = nullptr; r.n_rows = B; r.identity_tiles = 1;
    return launch_wgemm(WG_BF16_PLAIN, r, tiles, stream);
  }
  for (int b0 = 0; b0 < B; b0 += 8)
    if (int rc = launch_bf16_gemv_splitk(w, x + (size_t)b0 * cols, y + (size_t)b0 * rows, nullptr, rows, cols, std::min(8, B - b0), L->sk_ws,
                                         L->sk_bytes, stream))
      return rc;
  return BLOK_OK;
}

// The attention block for B entries (sequences, or the tokens of a prefill chunk): projections, cache append,
// attention, output projection.  Up to 8 entries: the split-K mat-vec kernels; 9..64: one pass of the weight-streaming
// kernel per projection (project()); the per-head products take every group of 8 entries in one launch.
static int decode_body(blok_mla_layer *L, const uint16_t *n, const CacheRef &c, const int *ctx_len, int B, uint16_t *out,
                       blok_stream_t stream_) {
  const blok_mla_weights &w = L->w;
  cudaStream_t stream = (cudaStream_t)stream_;
  const int lat_w = w.kv_rank + w.qk_rope, qk_head = w.qk_nope + w.qk_rope;
  const size_t q_row = (size_t)w.heads * qk_head, qf_row = (size_t)w.heads * lat_w, ol_row = (size_t)w.heads * w.kv_rank,
               av_row = (size_t)w.heads * w.v_head;
  int rc;
  const bool gemm = B > kWgStreamTokens;  // the GEMM form of the projections: needs the identity tile table
  const bool stream_rows = B > 8 && !gemm;  // 9..64 entries: one pass of the weight-streaming kernel per matrix
  if (gemm && (rc = launch_identity_tiles(B, L->tiles, L->tiles + L->n_tiles, L->tiles + 2 * L->n_tiles, L->tiles + 3 * L->n_tiles, stream)))
    return rc;
  // q_a -> RMSNorm -> q_b   (:813-815); kv_a (:816) reads the same activations as q_a and shares its launch where the
  // mat-vec kernel serves both (up to 8 entries per launch)
  if (!gemm && !stream_rows) {
    for (int b0 = 0; b0 < B; b0 += 8)
      if ((rc = launch_bf16_gemv_splitk_pair(w.q_a, w.q_rank, L->qa + (size_t)b0 * w.q_rank, w.kv_a, lat_w, L->kva + (size_t)b0 * lat_w,
                                             n + (size_t)b0 * w.hidden, w.hidden, std::min(8, B - b0), L->sk_ws, L->sk_bytes, stream)))
        return rc;
  } else {
    if ((rc = project(L, w.q_a, n, L->qa, w.q_rank, w.hidden, B, gemm, stream))) return rc;
    if ((rc = project(L, w.kv_a, n, L->kva, lat_w, w.hidden, B, gemm, stream))) return rc;
  }
  if ((rc = blok_rmsnorm(L->qa, w.q_a_ln, L->qa, B, w.q_rank, w.rms_eps, stream_))) return rc;
  if ((rc = project(L, w.q_b, L->qa, L->q, w.heads * qk_head, w.q_rank, B, gemm, stream))) return rc;
  // norm of c_kv, RoPE of k_pe and of q's rope part, cache append   (:816-824)
  mla_prep_kernel<<<dim3(1 + (w.heads * (w.qk_rope / 2) + 255) / 256, B), 256, 0, stream>>>(
      L->kva, w.kv_a_ln, L->q, L->inv_freq, ctx_len, c.base, c.seq_stride, L->q_full, L->seq, w.heads, w.qk_nope, w.qk_rope,
      w.kv_rank, w.rms_eps, c.block_table, c.slot_of, c.table_stride, c.page_rows, c.ctx_cap, L->err);
  if ((rc = launch_status("mla_prep_kernel"))) return rc;
  // q_abs = W_UK^T q_nope
  if ((rc = launch_head_gemv(L->wuk_t, (long)w.kv_rank * w.qk_nope, L->q, (long)q_row, qk_head, L->q_full, (long)qf_row, lat_w, w.kv_rank,
                             w.qk_nope, w.heads, B, stream)))
    return rc;
  if ((rc = attend_and_merge(L, L->q_full, c, L->seq, B, L->scale, L->o_lat, stream))) return rc;
  // out_h = W_UV o_lat_h, then o_proj   (:826)
  if ((rc = launch_head_gemv(w.kv_b + (size_t)w.qk_nope * w.kv_rank, (long)(w.qk_nope + w.v_head) * w.kv_rank, L->o_lat, (long)ol_row,
                             w.kv_rank, L->av, (long)av_row, w.v_head, w.v_head, w.kv_rank, w.heads, B, stream)))
    return rc;
  return project(L, w.o, L->av, out, w.hidden, w.heads * w.v_head, B, gemm, stream);
}

extern "C" int blok_mla_decode(blok_mla_layer_t *L, const blok_bf16_t *n, blok_bf16_t *cache, long ctx_stride,
                               const int *ctx_len, int B, blok_bf16_t *out, blok_stream_t stream_) {
  BLOK_REQUIRE(L && n && cache && ctx_len && out, BLOK_ERR_ARG, "blok_mla_decode: null pointer");
  BLOK_REQUIRE(B >= 1 && B <= L->max_batch && ctx_stride >= 1, BLOK_ERR_SHAPE, "blok_mla_decode: B=%d outside [1, %d]", B,
               L->max_batch);
  BLOK_REQUIRE((reinterpret_cast<uintptr_t>(n) & 15) == 0 && (reinterpret_cast<uintptr_t>(cache) & 15) == 0, BLOK_ERR_ARG,
               "blok_mla_decode: n and cache must be 16-byte aligned");
  CacheRef c;
  c.base = cache;
  c.seq_stride = c.ctx_cap = ctx_stride;
  return decode_body(L, n, c, ctx_len, B, out, stream_);
}

extern "C" int blok_mla_prefill(blok_mla_layer_t *L, const blok_bf16_t *n, blok_bf16_t *cache, long ctx_cap, const int *first_pos,
                                int T, blok_bf16_t *out, blok_stream_t stream_) {
  BLOK_REQUIRE(L && n && cache && first_pos && out, BLOK_ERR_ARG, "blok_mla_prefill: null pointer");
  BLOK_REQUIRE(T >= 1 && T <= L->max_batch && ctx_cap >= T, BLOK_ERR_SHAPE,
               "blok_mla_prefill: T=%d outside [1, %d] or larger than the cache (%ld rows)", T, L->max_batch, ctx_cap);
  BLOK_REQUIRE((reinterpret_cast<uintptr_t>(n) & 15) == 0 && (reinterpret_cast<uintptr_t>(cache) & 15) == 0, BLOK_ERR_ARG,
               "blok_mla_prefill: n and cache must be 16-byte aligned");
  mla_chunk_positions_kernel<<<(T + 63) / 64, 64, 0, (cudaStream_t)stream_>>>(first_pos, T, L->chunk_pos);
  if (int rc = launch_status("mla_chunk_positions_kernel")) return rc;
  CacheRef c;
  c.base = cache;
  c.seq_stride = 0;  // every token of the chunk appends to, and reads, the same sequence
  c.ctx_cap = ctx_cap;
  return decode_body(L, n, c, L->chunk_pos, T, out, stream_);
}

extern "C" int blok_mla_decode_paged(blok_mla_layer_t *L, const blok_bf16_t *n, blok_bf16_t *pool, const int *block_table,
                                     const int *slot_of, int table_stride, int page_rows, const int *ctx_len, int B,
                                     blok_bf16_t *out, blok_stream_t stream_) {
  BLOK_REQUIRE(L && n && ctx_len && out, BLOK_ERR_ARG, "blok_mla_decode_paged: null pointer");
  BLOK_REQUIRE(B >= 1 && B <= L->max_batch, BLOK_ERR_SHAPE, "blok_mla_decode_paged: B=%d outside [1, %d]", B, L->max_batch);
  BLOK_REQUIRE((reinterpret_cast<uintptr_t>(n) & 15) == 0, BLOK_ERR_ARG, "blok_mla_decode_paged: n must be 16-byte aligned");
  if (int rc = check_paged("blok_mla_decode_paged", pool, block_table, table_stride, page_rows)) return rc;
  CacheRef c;
  c.base = pool;
  c.ctx_cap = (long)table_stride * page_rows;
  c.block_table = block_table;
  c.slot_of = slot_of;
  c.table_stride = table_stride;
  c.page_rows = page_rows;
  return decode_body(L, n, c, ctx_len, B, out, stream_);
}
