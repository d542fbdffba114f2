// Router: fp32 logits, sigmoid, bias, top-k by repeated argmax, normalise, scale.
// Reference arithmetic: src/kimi_exec.cu:836-842 with matvec_bf16_f32_k :286-298,
// sigmoid_k :377-380, add_bf16_k :372-375, router_topk_k :382-397.
#include "router_topk.cuh"
#include "wgemm.h"

namespace blok {

int launch_bf16_gemv(const uint16_t *w, const uint16_t *x, uint16_t *y_bf16, float *y_f32, int rows, int cols, int T,
                     cudaStream_t stream);

constexpr int kTopkWarps = 4;

// One warp per token.  logits [T, experts] fp32.  The selection reproduces the
// reference's rule exactly: k rounds of argmax over sel = sigmoid(logit) + bias
// with strict '>' scanning ascending indices, i.e. the lowest index wins a tie,
// and the outputs are in descending sel order.
__global__ void router_topk_kernel(const float *__restrict__ logits, const float *__restrict__ bias, int T,
                                   int experts, int topk, float routed_scale, uint16_t *__restrict__ ids,
                                   float *__restrict__ wts, int *__restrict__ local_ids, int expert_base) {
  extern __shared__ float sm[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tok = blockIdx.x * kTopkWarps + warp;
  if (tok >= T) return;
  float *score = sm + (size_t)warp * 2 * experts;
  float *sel = score + experts;
  for (int i = lane; i < experts; i += 32) {
    float s = 1.0f / (1.0f + expf(-logits[(size_t)tok * experts + i]));
    score[i] = s;
    sel[i] = s + bias[i];
  }
  __syncwarp();
  int my_id;
  float my_w;
  warp_topk(score, sel, experts, topk, routed_scale, lane, my_id, my_w);
  if (lane < topk) {
    if (ids) ids[(size_t)tok * topk + lane] = (uint16_t)my_id;
    if (local_ids) local_ids[(size_t)tok * topk + lane] = my_id - expert_base;
    wts[(size_t)tok * topk + lane] = my_w;
  }
}

int launch_router_topk(const float *logits, const float *bias, int T, int experts, int topk, float routed_scale,
                       uint16_t *ids, float *wts, int *local_ids, int expert_base, cudaStream_t stream) {
  size_t smem = (size_t)kTopkWarps * 2 * experts * sizeof(float);
  router_topk_kernel<<<(T + kTopkWarps - 1) / kTopkWarps, kTopkWarps * 32, smem, stream>>>(logits, bias, T, experts,
                                                                                            topk, routed_scale, ids,
                                                                                            wts, local_ids,
                                                                                            expert_base);
  return launch_status("router_topk_kernel");
}

}  // namespace blok

using namespace blok;

// fp32 logits [T, experts], then (for more than 16 tokens) the tile table of the weight-streaming GEMM
static size_t router_logits_bytes(int T, int experts) { return ((size_t)T * experts * sizeof(float) + 255) / 256 * 256; }
extern "C" size_t blok_router_workspace_bytes(int T, int experts) {
  if (T <= 0 || experts <= 0) return 0;
  const size_t tiles = (size_t)(T + kWgTileTokens - 1) / kWgTileTokens;
  return router_logits_bytes(T, experts) + (3 * tiles + 1) * sizeof(int) + 256;
}

extern "C" int blok_router(const blok_bf16_t *router_w, const float *bias, const blok_bf16_t *x, int T, int experts,
                           int hidden, int topk, float routed_scale, uint16_t *ids, float *wts, void *workspace,
                           size_t workspace_bytes, blok_stream_t stream) {
  BLOK_REQUIRE(router_w && bias && x && ids && wts && workspace, BLOK_ERR_ARG, "blok_router: null pointer");
  BLOK_REQUIRE(T >= 0 && experts > 0 && experts <= 1024 && topk >= 1 && topk <= 32 && topk <= experts && hidden > 0 &&
                   hidden % 8 == 0,
               BLOK_ERR_SHAPE, "blok_router: unsupported shape T=%d experts=%d topk=%d hidden=%d", T, experts, topk, hidden);
  BLOK_REQUIRE(workspace_bytes >= blok_router_workspace_bytes(T, experts), BLOK_ERR_WORKSPACE,
               "blok_router: workspace too small");
  if (T == 0) return BLOK_OK;
  float *logits = static_cast<float *>(workspace);
  if (T > 16 && experts % 128 == 0 && hidden % 512 == 0) {
    // many tokens: one pass of the weight-streaming GEMM over the router matrix instead of T / 8 mat-vec launches
    const int tiles = (T + kWgTileTokens - 1) / kWgTileTokens;
    int *tab = reinterpret_cast<int *>(static_cast<unsigned char *>(workspace) + router_logits_bytes(T, experts));
    int rc = launch_identity_tiles(T, tab, tab + tiles, tab + 2 * tiles, tab + 3 * tiles, (cudaStream_t)stream);
    if (rc) return rc;
    WgArgs r;
    r.w_a = router_w; r.w_b = nullptr; r.s_a = r.s_b = nullptr; r.expert_stride_rows = 0; r.x = x; r.x_index = nullptr;
    r.K = hidden; r.R = experts; r.out_bf16 = nullptr; r.out_f32 = logits;
    r.tile_expert = tab; r.tile_start = tab + tiles; r.tile_count = tab + 2 * tiles; r.num_tiles = tab + 3 * tiles;
    r.out_index = nullptr; r.n_rows = T; r.identity_tiles = 1;
    if ((rc = launch_wgemm(WG_BF16_PLAIN, r, tiles, (cudaStream_t)stream))) return rc;
    return launch_router_topk(logits, bias, T, experts, topk, routed_scale, ids, wts, nullptr, 0, (cudaStream_t)stream);
  }
  for (int t0 = 0; t0 < T; t0 += 8) {
    int n = T - t0 < 8 ? T - t0 : 8;
    int rc = launch_bf16_gemv(router_w, x + (size_t)t0 * hidden, nullptr, logits + (size_t)t0 * experts, experts, hidden,
                              n, (cudaStream_t)stream);
    if (rc) return rc;
  }
  return launch_router_topk(logits, bias, T, experts, topk, routed_scale, ids, wts, nullptr, 0, (cudaStream_t)stream);
}
