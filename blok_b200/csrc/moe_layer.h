// Internal definition of the MoE layer handle (opaque in the C ABI).
#pragma once
#include <cstddef>
#include <cstdint>

#include "../../include/blok_b200.h"

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
};
