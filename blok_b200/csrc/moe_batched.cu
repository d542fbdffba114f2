// Batched routed-MoE layer: tokens are grouped by expert, every touched expert's
// INT4 weights are streamed once through the weight-streaming GEMM, and the
// per-assignment outputs are combined per token.  This is the per-token arithmetic
// of src/kimi_exec.cu:836-877 applied to T tokens; the reference itself only ever
// runs one token (:885-890).
#include <algorithm>

#include "common.cuh"
#include "moe_layer.h"
#include "wgemm.h"

namespace blok {

int launch_router_topk(const float *logits, const float *bias, int T, int experts, int topk, float routed_scale,
                       uint16_t *ids, float *wts, int *local_ids, int expert_base, cudaStream_t stream);

// counts[e] = assignments routed to local expert e; ids outside [0, n_local) are flagged in counts[n_local].
__global__ void mb_count_kernel(const int *__restrict__ expert_local, int N, int n_local, int *__restrict__ counts) {
  int a = blockIdx.x * blockDim.x + threadIdx.x;
  if (a >= N) return;
  int e = expert_local[a];
  if (e < 0 || e >= n_local) atomicAdd(counts + n_local, 1);
  else atomicAdd(counts + e, 1);
}

// One block: exclusive scan of the counts and the tile table (tiles of 64 sorted positions of one expert).
__global__ void __launch_bounds__(1024) mb_plan_kernel(const int *__restrict__ counts, int n_local, int *__restrict__ offsets,
                                                       int *__restrict__ tile_expert, int *__restrict__ tile_start,
                                                       int *__restrict__ tile_count, int *__restrict__ num_tiles, int max_tiles) {
  // one thread per expert (strided if there are more experts than threads); exclusive scans of the counts and of the
  // tiles per expert through shared memory: offsets and tiles come out in expert order, as a serial walk gives them
  __shared__ int s_off[1024], s_tiles[1024];
  __shared__ int s_base_off, s_base_tiles;
  const int tid = threadIdx.x, nth = blockDim.x;
  if (tid == 0) s_base_off = 0, s_base_tiles = 0;
  __syncthreads();
  for (int e0 = 0; e0 < n_local; e0 += nth) {
    const int e = e0 + tid;
    const int c = e < n_local ? counts[e] : 0;
    const int nt = (c + kWgTileTokens - 1) / kWgTileTokens;
    s_off[tid] = c;
    s_tiles[tid] = nt;
    __syncthreads();
    for (int d = 1; d < nth; d <<= 1) {  // inclusive scan (Hillis-Steele)
      const int a = tid >= d ? s_off[tid - d] : 0, t2 = tid >= d ? s_tiles[tid - d] : 0;
      __syncthreads();
      s_off[tid] += a;
      s_tiles[tid] += t2;
      __syncthreads();
    }
    const int off = s_base_off + s_off[tid] - c, first = s_base_tiles + s_tiles[tid] - nt;
    if (e < n_local) {
      offsets[e] = off;
      for (int k = 0; k < nt && first + k < max_tiles; ++k) {
        tile_expert[first + k] = e;
        tile_start[first + k] = off + k * kWgTileTokens;
        tile_count[first + k] = min(kWgTileTokens, c - k * kWgTileTokens);
      }
    }
    __syncthreads();
    if (tid == nth - 1) s_base_off += s_off[tid], s_base_tiles += s_tiles[tid];
    __syncthreads();
  }
  if (tid == 0) {
    offsets[n_local] = s_base_off;
    *num_tiles = min(s_base_tiles, max_tiles);
  }
}

// Identity tiles over T rows (a single group), for the shared expert and the router logits.
__global__ void mb_identity_tiles_kernel(int T, int *tile_expert, int *tile_start, int *tile_count, int *num_tiles) {
  int i = blockIdx.x * blockDim.x + threadIdx.x;
  int n = (T + kWgTileTokens - 1) / kWgTileTokens;
  if (i == 0) *num_tiles = n;
  if (i < n) {
    tile_expert[i] = 0;
    tile_start[i] = i * kWgTileTokens;
    tile_count[i] = min(kWgTileTokens, T - i * kWgTileTokens);
  }
}

int launch_identity_tiles(int T, int *tile_expert, int *tile_start, int *tile_count, int *num_tiles, cudaStream_t stream) {
  const int tt = (T + kWgTileTokens - 1) / kWgTileTokens;
  mb_identity_tiles_kernel<<<(tt + 63) / 64, 64, 0, stream>>>(T, tile_expert, tile_start, tile_count, num_tiles);
  return launch_status("mb_identity_tiles_kernel");
}

// One warp per local expert: stable placement (ascending assignment id) of its assignments.
__global__ void mb_scatter_kernel(const int *__restrict__ expert_local, const int *__restrict__ x_index, int N,
                                  int n_local, const int *__restrict__ offsets, int *__restrict__ sorted_assign,
                                  int *__restrict__ sorted_row) {
  const int e = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (e >= n_local) return;
  int pos = offsets[e];
  for (int a0 = 0; a0 < N; a0 += 32) {
    const int a = a0 + lane;
    const bool mine = a < N && expert_local[a] == e;
    const unsigned m = __ballot_sync(0xffffffffu, mine);
    if (mine) {
      const int p = pos + __popc(m & ((1u << lane) - 1));
      sorted_assign[p] = a;
      sorted_row[p] = x_index ? x_index[a] : a;
    }
    pos += __popc(m);
  }
}

__global__ void mb_assign_rows_kernel(int *rows, int N, int topk) {
  int a = blockIdx.x * blockDim.x + threadIdx.x;
  if (a < N) rows[a] = a / topk;
}

// out[t, c] = bf16( bf16(sum_k w[t,k] * y[t*topk + k, c]) + shared[t, c] ), slot order as :868-871, :684.
__global__ void mb_combine_kernel(const uint16_t *__restrict__ y, const float *__restrict__ wts,
                                  const uint16_t *__restrict__ shared, int hidden, int topk, uint16_t *__restrict__ out) {
  const int t = blockIdx.y;
  const int c = (blockIdx.x * blockDim.x + threadIdx.x) * 2;
  if (c >= hidden) return;
  float o0 = 0.f, o1 = 0.f;
  for (int k = 0; k < topk; ++k) {
    const uint32_t v = *reinterpret_cast<const uint32_t *>(y + ((size_t)t * topk + k) * hidden + c);
    const float w = wts[(size_t)t * topk + k];
    o0 = fmaf(bf16lo(v), w, o0);
    o1 = fmaf(bf16hi(v), w, o1);
  }
  o0 = round_bf16(o0);
  o1 = round_bf16(o1);
  if (shared) {
    const uint32_t s = *reinterpret_cast<const uint32_t *>(shared + (size_t)t * hidden + c);
    o0 = round_bf16(o0 + bf16lo(s));
    o1 = round_bf16(o1 + bf16hi(s));
  }
  *reinterpret_cast<uint32_t *>(out + (size_t)t * hidden + c) = pack_bf16x2(o0, o1);
}

static size_t al(size_t v) { return (v + 255) / 256 * 256; }

int batched_alloc(blok_moe_layer *L) {
  const blok_moe_weights &w = L->w;
  const size_t T = L->max_tokens, N = T * w.topk;
  const int nl = std::max(w.experts_local, 1);
  L->b_max_assign = (int)N;
  L->b_max_tiles = (int)((N + kWgTileTokens - 1) / kWgTileTokens) + nl;
  L->b_max_ttiles = (int)((std::max(T, N) + kWgTileTokens - 1) / kWgTileTokens);
  size_t off = 0;
  auto take = [&](size_t b) { size_t at = off; off = al(off + b); return at; };
  size_t o_counts = take((nl + 1) * 4), o_offsets = take((nl + 1) * 4), o_sa = take(N * 4), o_sr = take(N * 4);
  size_t o_te = take(L->b_max_tiles * 4), o_ts = take(L->b_max_tiles * 4), o_tc = take(L->b_max_tiles * 4), o_nt = take(8);  // the tile count, then the small-group kernel's limit
  size_t o_tte = take(L->b_max_ttiles * 4), o_tts = take(L->b_max_ttiles * 4), o_ttc = take(L->b_max_ttiles * 4), o_ntt = take(4);
  size_t o_ar = take(N * 4);
  size_t o_mid = take(N * (size_t)w.inter * 2), o_y = take(N * (size_t)w.hidden * 2);
  size_t o_smid = take(T * (size_t)std::max(w.shared_inter, 8) * 2), o_sout = take(T * (size_t)w.hidden * 2);
  // K-split partial sums of the bf16 products over a single tile of tokens (router, shared gate/up, shared down)
  const int rows_sk = (int)std::min<size_t>(T, 639);  // from 640 rows on the bf16 products take the tcgen05 kernel
  // (the router's 384 rows never do: its product is split at every token count the handle allows)
  L->b_splitk_bytes = std::max(wgemm_splitk_bytes(WG_BF16_PLAIN, w.hidden, w.experts, (int)T),
                               std::max(wgemm_splitk_bytes(WG_BF16_SWIGLU, w.hidden, std::max(w.shared_inter, 8), rows_sk),
                                        wgemm_splitk_bytes(WG_BF16_PLAIN, std::max(w.shared_inter, 8), w.hidden, rows_sk)));
  size_t o_sk = take(std::max(L->b_splitk_bytes, (size_t)16));
  BLOK_CUDA(cudaMalloc(&L->bws, off));
  unsigned char *b = static_cast<unsigned char *>(L->bws);
  L->b_counts = (int *)(b + o_counts); L->b_offsets = (int *)(b + o_offsets);
  L->b_sorted_assign = (int *)(b + o_sa); L->b_sorted_row = (int *)(b + o_sr);
  L->b_tile_expert = (int *)(b + o_te); L->b_tile_start = (int *)(b + o_ts); L->b_tile_count = (int *)(b + o_tc);
  L->b_num_tiles = (int *)(b + o_nt);
  L->b_ttile_expert = (int *)(b + o_tte); L->b_ttile_start = (int *)(b + o_tts); L->b_ttile_count = (int *)(b + o_ttc);
  L->b_num_ttiles = (int *)(b + o_ntt);
  L->b_assign_row = (int *)(b + o_ar);
  L->b_mid = (uint16_t *)(b + o_mid); L->b_y = (uint16_t *)(b + o_y);
  L->b_smid = (uint16_t *)(b + o_smid); L->b_sout = (uint16_t *)(b + o_sout);
  L->b_splitk = (float *)(b + o_sk);
  return BLOK_OK;
}

// y[a, :] = bf16(expert_{e_a}(x[row_a, :])) for N assignments; x_index NULL = identity.
int grouped_experts(blok_moe_layer *L, const uint16_t *x, const int *x_index, const int *expert_local, int N,
                    uint16_t *y, cudaStream_t stream) {
  const blok_moe_weights &w = L->w;
  const int nl = w.experts_local;
  BLOK_CUDA(cudaMemsetAsync(L->b_counts, 0, (nl + 1) * sizeof(int), stream));
  mb_count_kernel<<<(N + 255) / 256, 256, 0, stream>>>(expert_local, N, nl, L->b_counts);
  int rc = launch_status("mb_count_kernel");
  if (rc) return rc;
  mb_plan_kernel<<<1, 512, 0, stream>>>(L->b_counts, nl, L->b_offsets, L->b_tile_expert, L->b_tile_start, L->b_tile_count,
                                       L->b_num_tiles, L->b_max_tiles);
  if ((rc = launch_status("mb_plan_kernel"))) return rc;
  mb_scatter_kernel<<<(nl * 32 + 255) / 256, 256, 0, stream>>>(expert_local, x_index, N, nl, L->b_offsets,
                                                             L->b_sorted_assign, L->b_sorted_row);
  if ((rc = launch_status("mb_scatter_kernel"))) return rc;
  WgArgs g;
  g.w_a = w.gate_w; g.w_b = w.up_w; g.s_a = w.gate_s; g.s_b = w.up_s; g.expert_stride_rows = w.inter;
  g.x = x; g.x_index = L->b_sorted_row; g.K = w.hidden; g.R = w.inter; g.out_bf16 = L->b_mid; g.out_f32 = nullptr;
  g.tile_expert = L->b_tile_expert; g.tile_start = L->b_tile_start; g.tile_count = L->b_tile_count;
  g.num_tiles = L->b_num_tiles; g.out_index = nullptr; g.n_rows = N; g.small_limit = L->b_num_tiles + 1;
  const int max_tiles = std::min(L->b_max_tiles, (N + kWgTileTokens - 1) / kWgTileTokens + nl);
  if ((rc = launch_wgemm(WG_I4_SWIGLU, g, max_tiles, stream))) return rc;
  WgArgs d = g;
  d.w_a = w.down_w; d.w_b = nullptr; d.s_a = w.down_s; d.s_b = nullptr; d.expert_stride_rows = w.hidden;
  d.x = L->b_mid; d.x_index = nullptr; d.K = w.inter; d.R = w.hidden; d.out_bf16 = y; d.out_index = L->b_sorted_assign;
  return launch_wgemm(WG_I4_PLAIN, d, max_tiles, stream);
}

}  // namespace blok

using namespace blok;

extern "C" int blok_moe_experts_grouped(blok_moe_layer_t *L, const blok_bf16_t *x, const int *x_index,
                                        const int *expert_local, int N, blok_bf16_t *y, blok_stream_t stream) {
  BLOK_REQUIRE(L, BLOK_ERR_ARG, "blok_moe_experts_grouped: null layer");
  if (N == 0) return BLOK_OK;  // empty inputs may carry null pointers
  BLOK_REQUIRE(x && expert_local && y, BLOK_ERR_ARG, "blok_moe_experts_grouped: null pointer");
  BLOK_REQUIRE(L->bws, BLOK_ERR_STATE, "blok_moe_experts_grouped: the layer was created with max_tokens = 1");
  BLOK_REQUIRE(N >= 0 && N <= L->b_max_assign, BLOK_ERR_SHAPE, "blok_moe_experts_grouped: N=%d exceeds capacity %d", N,
               L->b_max_assign);
  BLOK_REQUIRE(L->w.hidden % 512 == 0 && L->w.inter % 512 == 0, BLOK_ERR_SHAPE,
               "blok_moe_experts_grouped: hidden and inter must be multiples of 512");
  if (N == 0) return BLOK_OK;
  return grouped_experts(L, x, x_index, expert_local, N, y, (cudaStream_t)stream);
}

extern "C" int blok_moe_batched(blok_moe_layer_t *L, const blok_bf16_t *x, int T, blok_bf16_t *y, uint16_t *ids_out,
                                float *wts_out, blok_stream_t stream_) {
  BLOK_REQUIRE(L && x && y, BLOK_ERR_ARG, "blok_moe_batched: null pointer");
  const blok_moe_weights &w = L->w;
  BLOK_REQUIRE(L->bws, BLOK_ERR_STATE, "blok_moe_batched: the layer was created with max_tokens = 1");
  BLOK_REQUIRE(T >= 0 && T <= L->max_tokens, BLOK_ERR_SHAPE, "blok_moe_batched: T=%d exceeds max_tokens %d", T, L->max_tokens);
  BLOK_REQUIRE(w.experts_local == w.experts && w.expert_base == 0, BLOK_ERR_ROUTE,
               "blok_moe_batched: needs every expert local; use blok_router + blok_moe_experts_grouped under expert parallelism");
  BLOK_REQUIRE(w.hidden % 512 == 0 && w.inter % 512 == 0 && w.experts % 128 == 0 && w.shared_inter % 512 == 0,
               BLOK_ERR_SHAPE, "blok_moe_batched: hidden/inter/shared_inter must be multiples of 512 and experts of 128");
  if (T == 0) return BLOK_OK;
  cudaStream_t stream = (cudaStream_t)stream_;
  const int N = T * w.topk;
  int rc;
  // router: logits through the weight-streaming GEMM (fp32, unrounded, :297), then the top-k kernel
  const int tt = (T + kWgTileTokens - 1) / kWgTileTokens;
  mb_identity_tiles_kernel<<<(tt + 63) / 64, 64, 0, stream>>>(T, L->b_ttile_expert, L->b_ttile_start, L->b_ttile_count,
                                                            L->b_num_ttiles);
  if ((rc = launch_status("mb_identity_tiles_kernel"))) return rc;
  WgArgs r;
  r.w_a = w.router_w; r.w_b = nullptr; r.s_a = r.s_b = nullptr; r.expert_stride_rows = 0; r.x = x; r.x_index = nullptr;
  r.K = w.hidden; r.R = w.experts; r.out_bf16 = nullptr; r.out_f32 = L->logits;
  r.tile_expert = L->b_ttile_expert; r.tile_start = L->b_ttile_start; r.tile_count = L->b_ttile_count;
  r.num_tiles = L->b_num_ttiles; r.out_index = nullptr; r.n_rows = T; r.identity_tiles = 1;
  r.splitk_ws = L->b_splitk; r.splitk_bytes = L->b_splitk_bytes;
  if ((rc = launch_wgemm(WG_BF16_PLAIN, r, tt, stream))) return rc;
  if ((rc = launch_router_topk(L->logits, w.router_bias, T, w.experts, w.topk, w.routed_scale, L->ids, L->wts, L->local_ids,
                               w.expert_base, stream)))
    return rc;
  mb_assign_rows_kernel<<<(N + 255) / 256, 256, 0, stream>>>(L->b_assign_row, N, w.topk);
  if ((rc = launch_status("mb_assign_rows_kernel"))) return rc;
  if ((rc = grouped_experts(L, x, L->b_assign_row, L->local_ids, N, L->b_y, stream))) return rc;
  const uint16_t *shared = nullptr;
  if (w.shared_inter > 0) {
    WgArgs s = r;
    s.w_a = w.shared_gate; s.w_b = w.shared_up; s.R = w.shared_inter; s.out_bf16 = L->b_smid; s.out_f32 = nullptr;
    if ((rc = launch_wgemm(WG_BF16_SWIGLU, s, tt, stream))) return rc;
    WgArgs d = r;
    d.w_a = w.shared_down; d.x = L->b_smid; d.K = w.shared_inter; d.R = w.hidden; d.out_bf16 = L->b_sout; d.out_f32 = nullptr;
    if ((rc = launch_wgemm(WG_BF16_PLAIN, d, tt, stream))) return rc;
    shared = L->b_sout;
  }
  mb_combine_kernel<<<dim3((w.hidden / 2 + 255) / 256, T), 256, 0, stream>>>(L->b_y, L->wts, shared, w.hidden, w.topk, y);
  if ((rc = launch_status("mb_combine_kernel"))) return rc;
  if (ids_out) BLOK_CUDA(cudaMemcpyAsync(ids_out, L->ids, (size_t)N * sizeof(uint16_t), cudaMemcpyDeviceToDevice, stream));
  if (wts_out) BLOK_CUDA(cudaMemcpyAsync(wts_out, L->wts, (size_t)N * sizeof(float), cudaMemcpyDeviceToDevice, stream));
  return BLOK_OK;
}

extern "C" int blok_moe_shared(blok_moe_layer_t *L, const blok_bf16_t *x, int T, blok_bf16_t *out, blok_stream_t stream_) {
  BLOK_REQUIRE(L && x && out, BLOK_ERR_ARG, "blok_moe_shared: null pointer");
  const blok_moe_weights &w = L->w;
  BLOK_REQUIRE(L->bws, BLOK_ERR_STATE, "blok_moe_shared: the layer was created with max_tokens = 1");
  BLOK_REQUIRE(w.shared_inter > 0 && w.shared_inter % 512 == 0 && w.hidden % 512 == 0, BLOK_ERR_SHAPE,
               "blok_moe_shared: needs a shared expert with sizes that are multiples of 512");
  BLOK_REQUIRE(T >= 0 && T <= L->max_tokens, BLOK_ERR_SHAPE, "blok_moe_shared: T=%d exceeds max_tokens %d", T, L->max_tokens);
  if (T == 0) return BLOK_OK;
  cudaStream_t stream = (cudaStream_t)stream_;
  const int tt = (T + kWgTileTokens - 1) / kWgTileTokens;
  mb_identity_tiles_kernel<<<(tt + 63) / 64, 64, 0, stream>>>(T, L->b_ttile_expert, L->b_ttile_start, L->b_ttile_count,
                                                            L->b_num_ttiles);
  int rc = launch_status("mb_identity_tiles_kernel");
  if (rc) return rc;
  WgArgs s;
  s.w_a = w.shared_gate; s.w_b = w.shared_up; s.s_a = s.s_b = nullptr; s.expert_stride_rows = 0; s.x = x; s.x_index = nullptr;
  s.K = w.hidden; s.R = w.shared_inter; s.out_bf16 = L->b_smid; s.out_f32 = nullptr;
  s.tile_expert = L->b_ttile_expert; s.tile_start = L->b_ttile_start; s.tile_count = L->b_ttile_count;
  s.num_tiles = L->b_num_ttiles; s.out_index = nullptr; s.n_rows = T; s.identity_tiles = 1;
  s.splitk_ws = L->b_splitk; s.splitk_bytes = L->b_splitk_bytes;
  if ((rc = launch_wgemm(WG_BF16_SWIGLU, s, tt, stream))) return rc;
  WgArgs d = s;
  d.w_a = w.shared_down; d.w_b = nullptr; d.x = L->b_smid; d.K = w.shared_inter; d.R = w.hidden; d.out_bf16 = out;
  return launch_wgemm(WG_BF16_PLAIN, d, tt, stream);
}

extern "C" int blok_moe_combine(const blok_bf16_t *y_assign, const float *wts, const blok_bf16_t *shared, int T, int topk,
                                int hidden, blok_bf16_t *out, blok_stream_t stream) {
  BLOK_REQUIRE(y_assign && wts && out, BLOK_ERR_ARG, "blok_moe_combine: null pointer");
  BLOK_REQUIRE(T >= 0 && topk >= 1 && hidden > 0 && hidden % 2 == 0, BLOK_ERR_SHAPE, "blok_moe_combine: bad shape");
  if (T == 0) return BLOK_OK;
  mb_combine_kernel<<<dim3((hidden / 2 + 255) / 256, T), 256, 0, (cudaStream_t)stream>>>(y_assign, wts, shared, hidden, topk,
                                                                                        out);
  return launch_status("mb_combine_kernel");
}
