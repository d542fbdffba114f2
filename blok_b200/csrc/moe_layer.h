// Internal definition of the MoE layer handle (opaque in the C ABI).
#pragma once
#include <cstddef>
#include <cstdint>

#include "../../include/blok_b200.h"

namespace blok {
// Launch geometry and scratch sizing of the fused decode kernel (moe_fused.cu).
struct FusedPlan {
  bool enabled = false;
  int grid = 0;
  size_t smem = 0;
  int total_warps = 0;
  // row-blocks per phase; steps per row-block, steps per chunk, chunks per row-block
  int nrbR = 0, nrbA = 0, nrbB = 0, nrbC1 = 0, nrbC2 = 0;
  int sprR = 0, spcR = 0, cprR = 1;
  int sprA = 0, spcA = 0, cprA = 1;
  int sprB = 0, spcB = 0, cprB = 1;
  int sprC1 = 0;
  int sprC2 = 0, spcC2 = 0, cprC2 = 1;
};
}  // namespace blok

struct blok_moe_layer {
  blok_moe_weights w;
  int max_tokens = 0;
  void *ws = nullptr;
  size_t ws_bytes = 0;
  // decode workspace (views into ws)
  float *logits = nullptr;       // [max_tokens, experts]
  uint16_t *ids = nullptr;       // [max_tokens, topk] global expert ids
  int *local_ids = nullptr;      // [max_tokens, topk] id - expert_base
  float *wts = nullptr;          // [max_tokens, topk]
  uint16_t *mid = nullptr;       // [topk, inter] bf16
  uint16_t *shared_mid = nullptr;  // [8, shared_inter]
  uint16_t *shared_out = nullptr;  // [8, hidden]
  uint16_t *io_x = nullptr;        // [hidden] staging for the host-buffer entry point
  uint16_t *io_y = nullptr;        // [hidden]
  unsigned *io_err_host = nullptr; // pinned: the fused kernel's error word, written by the kernel's last CTA in host-buffer calls
  const void *io_last_host = nullptr;  // the host buffer last asked about, and its device address (NULL: not pinned)
  void *io_last_dev = nullptr;
  // batched path (moe_batched.cu); allocated when max_tokens > 1
  void *bws = nullptr;
  int b_max_assign = 0;          // max_tokens * topk
  int b_max_tiles = 0, b_max_ttiles = 0;
  int *b_counts = nullptr;       // [experts_local + 1]
  int *b_offsets = nullptr;      // [experts_local + 1]
  int *b_sorted_assign = nullptr;  // [N] assignment id at sorted position p
  int *b_sorted_row = nullptr;     // [N] x row at sorted position p
  int *b_tile_expert = nullptr, *b_tile_start = nullptr, *b_tile_count = nullptr, *b_num_tiles = nullptr;
  int *b_ttile_expert = nullptr, *b_ttile_start = nullptr, *b_ttile_count = nullptr, *b_num_ttiles = nullptr;
  int *b_assign_row = nullptr;   // [N] token row of assignment a (a / topk)
  uint16_t *b_mid = nullptr;     // [N, inter] sorted order
  uint16_t *b_y = nullptr;       // [N, hidden] assignment order
  uint16_t *b_smid = nullptr;    // [T, shared_inter]
  uint16_t *b_sout = nullptr;    // [T, hidden]
  float *b_splitk = nullptr;     // K-split partial sums of the bf16 products over one tile of tokens
  size_t b_splitk_bytes = 0;
  // fused decode kernel scratch
  blok::FusedPlan plan;
  bool use_fused = false;
  uint16_t *f_mid = nullptr;  // [topk + 1][f_mid_stride / 2] tagged pairs (8 bytes each)
  float *f_logits_t = nullptr;  // [experts] tagged logits (8 bytes each)
  int f_mid_stride = 0;
  float *f_ys = nullptr;      // [topk + 1][hidden]
  float *f_partR = nullptr, *f_partA = nullptr, *f_partB = nullptr, *f_partC2 = nullptr;
  unsigned *f_cntR = nullptr, *f_cntA = nullptr, *f_cntB = nullptr, *f_cntC2 = nullptr, *f_cntOut = nullptr;
  unsigned *f_ctrl = nullptr;  // [8] queue head, router row-blocks, routed, mid row-blocks, exits, error
  int *f_route_ids = nullptr;   // [16]
  float *f_route_wts = nullptr; // [16]
  long long *f_trace = nullptr;  // [1 + grid][16] time stamps, only with BLOK_MOE_TRACE=1
  void *f_counters = nullptr;  // start of the counter block (zeroed on reset)
  size_t f_counters_bytes = 0;
};
