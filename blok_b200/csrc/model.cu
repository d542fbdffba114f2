// Whole-model decode step and greedy generation.  Reference: generate() and its
// `run` lambda, src/kimi_exec.cu:780-893 (per-layer body :803-878, sampler :880-881,
// prompt replay and decode loop :885-890).  Weights are resident in HBM; the
// reference re-reads every tile from storage on every use (:608-649).
#include <algorithm>
#include <cstring>
#include <map>
#include <new>
#include <string>
#include <vector>

#include "common.cuh"
#include "wgemm.h"

namespace blok {

// ---- seeded synthetic weights: a counter-based generator, one value per element --------------
__device__ __forceinline__ uint64_t mix64(uint64_t z) {
  z += 0x9e3779b97f4a7c15ull;
  z = (z ^ (z >> 30)) * 0xbf58476d1ce4e5b9ull;
  z = (z ^ (z >> 27)) * 0x94d049bb133111ebull;
  return z ^ (z >> 31);
}
__device__ __forceinline__ float unit_normal(uint64_t key, uint64_t i) {
  uint64_t r = mix64(key ^ mix64(i));
  float u1 = ((uint32_t)(r >> 40) + 1.0f) * (1.0f / 16777217.0f);  // (0, 1)
  float u2 = (uint32_t)(r & 0xffffff) * (1.0f / 16777216.0f);
  return sqrtf(-2.0f * logf(u1)) * cosf(6.28318530718f * u2);
}

// `first` is the index, in the whole tensor, of the first element generated: a rank's shard of the experts holds exactly
// the values the unsharded tensor has at those positions.
__global__ void fill_words_kernel(uint32_t *p, size_t n, uint64_t key, size_t first) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) p[i] = (uint32_t)mix64(key ^ mix64(i + first));
}
// mode 0: N(0, std); mode 1: |N(0, std)|; mode 2: constant std
__global__ void fill_bf16_kernel(uint16_t *p, size_t n, uint64_t key, float std, int mode, size_t first) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  float v = mode == 2 ? std : unit_normal(key, i + first) * std;
  if (mode == 1) v = fabsf(v);
  p[i] = f32_to_bf16_bits(v);
}
__global__ void fill_f32_kernel(float *p, size_t n, uint64_t key, float std) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) p[i] = unit_normal(key, i) * std;
}
__global__ void advance_kernel(int *pos, int n, int by) {
  int i = threadIdx.x;
  if (i < n) pos[i] += by;
}

constexpr int kMaxBatch = 64;  // sequences per step, and tokens per prefill chunk

// Paged model: batch entry b is the sequence in slot slot_of[b].
__global__ void gather_positions_kernel(const int *__restrict__ pos, const int *__restrict__ slot_of, int n, int *__restrict__ ctx) {
  const int b = threadIdx.x;
  if (b < n) ctx[b] = pos[slot_of[b]];
}
__global__ void advance_slots_kernel(int *__restrict__ pos, const int *__restrict__ slot_of, int n) {
  const int b = threadIdx.x;
  if (b < n) pos[slot_of[b]] += 1;  // the slots of a step are distinct
}
// A prompt chunk of the sequence in `slot`: entry i is that slot at position pos[slot] + i.
__global__ void chunk_slots_kernel(const int *__restrict__ pos, int slot, int n, int *__restrict__ ctx, int *__restrict__ slot_of) {
  const int i = threadIdx.x;
  if (i < n) {
    ctx[i] = pos[slot] + i;
    slot_of[i] = slot;
  }
}

// Expert-parallel decode (every rank holds the same rows): the weighted sum of the selected experts THIS rank holds,
// unrounded, rows of experts held elsewhere skipped; the ranks' sums are added by one all-reduce per layer.
__global__ void sharded_partial_kernel(const uint16_t *__restrict__ y_assign, const float *__restrict__ wts,
                                       const int *__restrict__ local_ids, int n_local, int hidden, int topk, float *__restrict__ part) {
  const int t = blockIdx.y;
  const int c = (blockIdx.x * blockDim.x + threadIdx.x) * 2;
  if (c >= hidden) return;
  float o0 = 0.f, o1 = 0.f;
  for (int k = 0; k < topk; ++k) {
    const int e = local_ids[(size_t)t * topk + k];
    if (e < 0 || e >= n_local) continue;
    const uint32_t v = *reinterpret_cast<const uint32_t *>(y_assign + ((size_t)t * topk + k) * hidden + c);
    const float w = wts[(size_t)t * topk + k];
    o0 = fmaf(bf16lo(v), w, o0);
    o1 = fmaf(bf16hi(v), w, o1);
  }
  *reinterpret_cast<float2 *>(part + (size_t)t * hidden + c) = make_float2(o0, o1);
}
// out = bf16(bf16(routed sum) + shared), the rounding points of src/kimi_exec.cu:871 and :684.
__global__ void sharded_finish_kernel(const float *__restrict__ part, const uint16_t *__restrict__ shared, int hidden,
                                      uint16_t *__restrict__ out) {
  const int t = blockIdx.y;
  const int c = (blockIdx.x * blockDim.x + threadIdx.x) * 2;
  if (c >= hidden) return;
  const float2 v = *reinterpret_cast<const float2 *>(part + (size_t)t * hidden + c);
  float o0 = round_bf16(v.x), o1 = round_bf16(v.y);
  if (shared) {
    const uint32_t s = *reinterpret_cast<const uint32_t *>(shared + (size_t)t * hidden + c);
    o0 = round_bf16(o0 + bf16lo(s));
    o1 = round_bf16(o1 + bf16hi(s));
  }
  *reinterpret_cast<uint32_t *>(out + (size_t)t * hidden + c) = pack_bf16x2(o0, o1);
}

int launch_bf16_gemv(const uint16_t *w, const uint16_t *x, uint16_t *y_bf16, float *y_f32, int rows, int cols, int T,
                     cudaStream_t stream);
int launch_router_topk(const float *logits, const float *bias, int T, int experts, int topk, float routed_scale,
                       uint16_t *ids, float *wts, int *local_ids, int expert_base, cudaStream_t stream);

struct Tensor {
  void *ptr = nullptr;
  size_t bytes = 0;
};

struct LayerWeights {
  std::map<std::string, Tensor> t;
  blok_mla_layer_t *mla = nullptr;
  blok_moe_layer_t *moe = nullptr;
  uint16_t *cache = nullptr;  // [max_batch, max_ctx, kv_rank + qk_rope], or the page pool [kv_pages, kv_page_rows, ...]
};

}  // namespace blok

struct blok_model {
  blok_model_config cfg;
  std::vector<blok::LayerWeights> layers;
  std::map<std::string, blok::Tensor> top;
  std::vector<void *> allocations;
  // step buffers
  uint16_t *x = nullptr, *n = nullptr, *tmp = nullptr;  // [max(max_batch, prefill_chunk), hidden]
  uint32_t *prompt_ids = nullptr;                       // [max(max_ctx, rows)] token ids given on the host (prefill_chunk >= 1)
  int rows = 0;                                         // max(max_batch, prefill_chunk)
  bool moe_batched_ok = false;                          // the layer sizes fit the grouped-GEMM kernels
  std::vector<long> host_pos;                           // tokens cached per sequence (host mirror of pos)
  // paged cache (cfg.kv_page_rows > 0): one table for all layers' pools
  blok_kv_pages_t *pages = nullptr;
  int table_stride = 0;
  int *table_dev = nullptr;                             // [max_batch, table_stride]
  int *slot_of = nullptr, *ctx_b = nullptr;             // [rows] slot and position of every batch entry of the call in flight
  int *pos = nullptr;                                   // [max_batch]
  uint32_t *ids = nullptr, *next = nullptr;             // [max_batch]
  void *mlp_ws = nullptr;
  size_t mlp_ws_bytes = 0;
  int mlp_rows = 8;            // rows of the dense layer per call
  void *head_ws = nullptr;
  size_t head_ws_bytes = 0;
  uint64_t seed = 0, counter = 0;
  // One CUDA graph of the whole step per batch size: a step is ~16 small launches per layer and the host cannot issue
  // them as fast as the GPU runs them.  steps_seen counts eager steps (the first one also sets kernel attributes).
  cudaGraphExec_t step_graph[blok::kMaxBatch + 1] = {};
  long long graph_launches[blok::kMaxBatch + 1] = {};  // kernels in each graph, added to the launch counter at every replay
  int steps_seen[blok::kMaxBatch + 1] = {};
  bool graphs_enabled = true;
  // expert parallelism (cfg.ep_world > 1): this rank holds experts [ep_base, ep_base + ep_local) of every MoE layer
  blok_comm_t *comm = nullptr;
  int ep_base = 0, ep_local = 0;
  float *ep_logits = nullptr;   // [rows, experts]
  float *ep_sk = nullptr;       // K-split partial sums of the router logits over 9..64 rows
  size_t ep_sk_bytes = 0;
  uint16_t *ep_ids = nullptr;   // [rows, topk]
  int *ep_local_ids = nullptr;  // [rows, topk] id - ep_base (outside [0, ep_local): held by another rank)
  int *ep_rows = nullptr;       // [rows * topk] row of assignment a: a / topk
  float *ep_wts = nullptr;      // [rows, topk]
  uint16_t *ep_y = nullptr;     // [rows * topk, hidden] outputs of the assignments held here
  float *ep_part = nullptr;     // [rows, hidden] this rank's weighted sum, then the sum over the ranks
  uint16_t *ep_shared = nullptr;  // [rows, hidden]
};

using namespace blok;

namespace {

int dev_alloc(blok_model *m, size_t bytes, void **out) {
  void *p = nullptr;
  BLOK_CUDA(cudaMalloc(&p, bytes ? bytes : 16));
  m->allocations.push_back(p);
  *out = p;
  return BLOK_OK;
}

enum Fill { F_NORMAL, F_ABS, F_ONE, F_WORDS, F_F32 };

int make_tensor(blok_model *m, std::map<std::string, Tensor> &into, const char *name, size_t elems, Fill fill, float std,
                size_t first = 0) {
  size_t esz = (fill == F_WORDS || fill == F_F32) ? 4 : 2;
  Tensor t;
  t.bytes = elems * esz;
  int rc = dev_alloc(m, t.bytes, &t.ptr);
  if (rc) return rc;
  const uint64_t key = m->seed * 0x100000001b3ull + (++m->counter) * 0x9e3779b97f4a7c15ull;
  const unsigned blocks = (unsigned)((elems + 255) / 256);
  if (elems) {
    if (fill == F_WORDS) fill_words_kernel<<<blocks, 256>>>(static_cast<uint32_t *>(t.ptr), elems, key, first);
    else if (fill == F_F32) fill_f32_kernel<<<blocks, 256>>>(static_cast<float *>(t.ptr), elems, key, std);
    else fill_bf16_kernel<<<blocks, 256>>>(static_cast<uint16_t *>(t.ptr), elems, key, fill == F_ONE ? 1.0f : std,
                                           fill == F_ONE ? 2 : (fill == F_ABS ? 1 : 0), first);
    rc = launch_status("synthetic fill");
    if (rc) return rc;
  }
  into[name] = t;
  return BLOK_OK;
}

template <typename T>
T *tp(const std::map<std::string, Tensor> &m, const char *name) {
  auto it = m.find(name);
  return it == m.end() ? nullptr : static_cast<T *>(it->second.ptr);
}

int build(blok_model *m) {
  const blok_model_config &c = m->cfg;
  m->rows = c.max_batch > c.prefill_chunk ? c.max_batch : c.prefill_chunk;
  const int world = c.ep_world > 1 ? c.ep_world : 1;
  m->ep_local = c.experts / world;
  m->ep_base = (world > 1 ? c.ep_rank : 0) * m->ep_local;
  // the grouped-GEMM form of the MoE layer (blok_moe_batched) serves prefill chunks and steps of more than 8 sequences
  m->moe_batched_ok = m->rows > 1 && c.first_dense < c.layers && c.hidden % 512 == 0 && c.inter % 512 == 0 &&
                      c.experts % 128 == 0 && c.shared_inter % 512 == 0;
  const size_t H = c.hidden;
  const float wstd = 0.006f;
  int rc;
#define MK(map, name, elems, fill, std) \
  if ((rc = make_tensor(m, map, name, (size_t)(elems), fill, std))) return rc;
  MK(m->top, "embed_tokens", (size_t)c.vocab * H, F_NORMAL, wstd);
  MK(m->top, "norm", H, F_ONE, 1.f);
  MK(m->top, "lm_head", (size_t)c.vocab * H, F_NORMAL, wstd);
  m->layers.resize(c.layers);
  const int qk_head = c.qk_nope + c.qk_rope, lat_w = c.kv_rank + c.qk_rope;
  for (int l = 0; l < c.layers; ++l) {
    auto &t = m->layers[l].t;
    MK(t, "input_layernorm", H, F_ONE, 1.f);
    MK(t, "post_attention_layernorm", H, F_ONE, 1.f);
    MK(t, "q_a_proj", (size_t)c.q_rank * H, F_NORMAL, wstd);
    MK(t, "q_a_layernorm", c.q_rank, F_ONE, 1.f);
    MK(t, "q_b_proj", (size_t)c.heads * qk_head * c.q_rank, F_NORMAL, wstd);
    MK(t, "kv_a_proj_with_mqa", (size_t)lat_w * H, F_NORMAL, wstd);
    MK(t, "kv_a_layernorm", c.kv_rank, F_ONE, 1.f);
    MK(t, "kv_b_proj", (size_t)c.heads * (c.qk_nope + c.v_head) * c.kv_rank, F_NORMAL, wstd);
    MK(t, "o_proj", H * (size_t)c.heads * c.v_head, F_NORMAL, wstd);
    if (l < c.first_dense) {
      MK(t, "gate_proj", (size_t)c.dense_inter * H, F_NORMAL, wstd);
      MK(t, "up_proj", (size_t)c.dense_inter * H, F_NORMAL, wstd);
      MK(t, "down_proj", H * (size_t)c.dense_inter, F_NORMAL, wstd);
    } else {
      const size_t E = c.experts, I = c.inter;
      const size_t El = m->ep_local, E0 = m->ep_base;  // this rank's experts; the values are those of the whole tensor
      MK(t, "router", E * H, F_NORMAL, wstd);
      MK(t, "router_bias", E, F_F32, 0.01f);
#define MKE(name, per_expert, fill, std) \
  if ((rc = make_tensor(m, t, name, El * (size_t)(per_expert), fill, std, E0 * (size_t)(per_expert)))) return rc;
      MKE("gate_w", I * (H / 8), F_WORDS, 0.f);
      MKE("gate_s", I * (H / 32), F_ABS, 0.003f);
      MKE("up_w", I * (H / 8), F_WORDS, 0.f);
      MKE("up_s", I * (H / 32), F_ABS, 0.003f);
      MKE("down_w", H * (I / 8), F_WORDS, 0.f);
      MKE("down_s", H * (I / 32), F_ABS, 0.003f);
#undef MKE
      if (c.shared_inter) {
        MK(t, "shared_gate", (size_t)c.shared_inter * H, F_NORMAL, wstd);
        MK(t, "shared_up", (size_t)c.shared_inter * H, F_NORMAL, wstd);
        MK(t, "shared_down", H * (size_t)c.shared_inter, F_NORMAL, wstd);
      }
    }
    void *cache = nullptr;
    const size_t cache_rows = c.kv_page_rows > 0 ? (size_t)c.kv_pages * c.kv_page_rows : (size_t)c.max_batch * c.max_ctx;
    if ((rc = dev_alloc(m, cache_rows * lat_w * 2, &cache))) return rc;
    m->layers[l].cache = static_cast<uint16_t *>(cache);
  }
#undef MK
  BLOK_CUDA(cudaDeviceSynchronize());
  for (int l = 0; l < c.layers; ++l) {
    auto &L = m->layers[l];
    blok_mla_weights mw;
    memset(&mw, 0, sizeof(mw));
    mw.hidden = c.hidden; mw.heads = c.heads; mw.qk_nope = c.qk_nope; mw.qk_rope = c.qk_rope; mw.v_head = c.v_head;
    mw.q_rank = c.q_rank; mw.kv_rank = c.kv_rank; mw.rms_eps = c.rms_eps; mw.rope_theta = c.rope_theta;
    mw.yarn_factor = c.yarn_factor; mw.yarn_beta_fast = c.yarn_beta_fast; mw.yarn_beta_slow = c.yarn_beta_slow;
    mw.yarn_original_ctx = c.yarn_original_ctx; mw.yarn_mscale_all_dim = c.yarn_mscale_all_dim;
    mw.q_a = tp<uint16_t>(L.t, "q_a_proj"); mw.q_a_ln = tp<uint16_t>(L.t, "q_a_layernorm");
    mw.q_b = tp<uint16_t>(L.t, "q_b_proj"); mw.kv_a = tp<uint16_t>(L.t, "kv_a_proj_with_mqa");
    mw.kv_a_ln = tp<uint16_t>(L.t, "kv_a_layernorm"); mw.kv_b = tp<uint16_t>(L.t, "kv_b_proj");
    mw.o = tp<uint16_t>(L.t, "o_proj");
    if ((rc = blok_mla_layer_create(&mw, m->rows, c.max_ctx, &L.mla))) return rc;
    if (l >= c.first_dense) {
      blok_moe_weights ew;
      memset(&ew, 0, sizeof(ew));
      ew.hidden = c.hidden; ew.inter = c.inter; ew.experts = c.experts; ew.topk = c.topk; ew.shared_inter = c.shared_inter;
      ew.routed_scale = c.routed_scale; ew.router_w = tp<uint16_t>(L.t, "router");
      ew.router_bias = tp<float>(L.t, "router_bias"); ew.expert_base = m->ep_base; ew.experts_local = m->ep_local;
      ew.gate_w = tp<uint32_t>(L.t, "gate_w"); ew.gate_s = tp<uint16_t>(L.t, "gate_s");
      ew.up_w = tp<uint32_t>(L.t, "up_w"); ew.up_s = tp<uint16_t>(L.t, "up_s");
      ew.down_w = tp<uint32_t>(L.t, "down_w"); ew.down_s = tp<uint16_t>(L.t, "down_s");
      ew.shared_gate = tp<uint16_t>(L.t, "shared_gate"); ew.shared_up = tp<uint16_t>(L.t, "shared_up");
      ew.shared_down = tp<uint16_t>(L.t, "shared_down");
      // a sharded layer always runs its experts through the grouped kernels, which need the batched scratch
      const int moe_rows = world > 1 ? (m->rows > 2 ? m->rows : 2) : (m->moe_batched_ok ? m->rows : 1);
      if ((rc = blok_moe_layer_create(&ew, moe_rows, &L.moe))) return rc;
    }
  }
  void *p;
  const size_t act = (size_t)m->rows * c.hidden * 2;
  if ((rc = dev_alloc(m, act, &p))) return rc; m->x = static_cast<uint16_t *>(p);
  if ((rc = dev_alloc(m, act, &p))) return rc; m->n = static_cast<uint16_t *>(p);
  if ((rc = dev_alloc(m, act, &p))) return rc; m->tmp = static_cast<uint16_t *>(p);
  if ((rc = dev_alloc(m, c.max_batch * 4, &p))) return rc; m->pos = static_cast<int *>(p);
  if ((rc = dev_alloc(m, m->rows * 4, &p))) return rc; m->ids = static_cast<uint32_t *>(p);
  if ((rc = dev_alloc(m, m->rows * 4, &p))) return rc; m->next = static_cast<uint32_t *>(p);
  if ((rc = dev_alloc(m, (size_t)(c.prefill_chunk > 0 ? (c.max_ctx > m->rows ? c.max_ctx : m->rows) : 1) * 4, &p))) return rc;
  m->prompt_ids = static_cast<uint32_t *>(p);
  // the dense layer takes up to 64 rows per call where its sizes fit the weight-streaming kernel, else 8
  m->mlp_rows = (c.hidden % 256 == 0 && c.dense_inter % 256 == 0 && c.dense_inter > 0) ? std::min((int)m->rows, kWgStreamTokens) : 8;
  m->mlp_ws_bytes = blok_bf16_mlp_workspace_bytes(c.hidden, c.dense_inter > 0 ? c.dense_inter : 32, std::max(m->mlp_rows, 8));
  if ((rc = dev_alloc(m, m->mlp_ws_bytes, &m->mlp_ws))) return rc;
  m->head_ws_bytes = blok_lm_head_workspace_bytes(c.vocab, c.max_batch);
  if ((rc = dev_alloc(m, m->head_ws_bytes, &m->head_ws))) return rc;
  if (world > 1) {
    if ((rc = dev_alloc(m, (size_t)m->rows * c.experts * 4, &p))) return rc; m->ep_logits = static_cast<float *>(p);
    m->ep_sk_bytes = wgemm_splitk_bytes(WG_BF16_PLAIN, c.hidden, c.experts, std::min((int)m->rows, kWgStreamTokens));
    if ((rc = dev_alloc(m, std::max(m->ep_sk_bytes, (size_t)16), &p))) return rc; m->ep_sk = static_cast<float *>(p);
    if ((rc = dev_alloc(m, (size_t)m->rows * c.topk * 2, &p))) return rc; m->ep_ids = static_cast<uint16_t *>(p);
    if ((rc = dev_alloc(m, (size_t)m->rows * c.topk * 4, &p))) return rc; m->ep_local_ids = static_cast<int *>(p);
    if ((rc = dev_alloc(m, (size_t)m->rows * c.topk * 4, &p))) return rc; m->ep_wts = static_cast<float *>(p);
    if ((rc = dev_alloc(m, (size_t)m->rows * c.topk * 4, &p))) return rc; m->ep_rows = static_cast<int *>(p);
    {
      std::vector<int> rows_of((size_t)m->rows * c.topk);
      for (size_t a = 0; a < rows_of.size(); ++a) rows_of[a] = (int)(a / c.topk);
      BLOK_CUDA(cudaMemcpy(m->ep_rows, rows_of.data(), rows_of.size() * 4, cudaMemcpyHostToDevice));
    }
    if ((rc = dev_alloc(m, (size_t)m->rows * c.topk * c.hidden * 2, &p))) return rc; m->ep_y = static_cast<uint16_t *>(p);
    if ((rc = dev_alloc(m, (size_t)m->rows * c.hidden * 4, &p))) return rc; m->ep_part = static_cast<float *>(p);
    if ((rc = dev_alloc(m, (size_t)m->rows * c.hidden * 2, &p))) return rc; m->ep_shared = static_cast<uint16_t *>(p);
  }
  BLOK_CUDA(cudaMemset(m->pos, 0, c.max_batch * 4));
  m->host_pos.assign(c.max_batch, 0);
  if (c.kv_page_rows > 0) {
    m->table_stride = (c.max_ctx + c.kv_page_rows - 1) / c.kv_page_rows;
    if ((rc = blok_kv_pages_create(c.kv_pages, c.kv_page_rows, c.max_batch, m->table_stride, &m->pages))) return rc;
    if ((rc = dev_alloc(m, (size_t)c.max_batch * m->table_stride * 4, &p))) return rc; m->table_dev = static_cast<int *>(p);
    BLOK_CUDA(cudaMemset(m->table_dev, 0, (size_t)c.max_batch * m->table_stride * 4));
    if ((rc = dev_alloc(m, m->rows * 4, &p))) return rc; m->slot_of = static_cast<int *>(p);
    if ((rc = dev_alloc(m, m->rows * 4, &p))) return rc; m->ctx_b = static_cast<int *>(p);
  }
  return BLOK_OK;
}

}  // namespace

extern "C" void blok_model_default_config(blok_model_config *c) {
  if (!c) return;
  memset(c, 0, sizeof(*c));
  c->layers = 61; c->first_dense = 1; c->hidden = 7168; c->vocab = 163840; c->dense_inter = 18432;
  c->inter = 2048; c->experts = 384; c->topk = 8; c->shared_inter = 2048; c->routed_scale = 2.827f;
  c->heads = 64; c->qk_nope = 128; c->qk_rope = 64; c->v_head = 128; c->q_rank = 1536; c->kv_rank = 512;
  c->rms_eps = 1.0e-5f; c->final_rms_eps = 1.0e-5f;
  c->rope_theta = 50000.0f; c->yarn_factor = 64.0f; c->yarn_beta_fast = 32.0f; c->yarn_beta_slow = 1.0f;
  c->yarn_original_ctx = 4096.0f; c->yarn_mscale_all_dim = 1.0f;
  c->max_batch = 1; c->max_ctx = 1024; c->eos_id = 163586u;
}

extern "C" int blok_model_destroy(blok_model_t *m) {
  if (m)
    for (auto &g : m->step_graph)
      if (g) cudaGraphExecDestroy(g);
  if (!m) return BLOK_OK;
  blok_kv_pages_destroy(m->pages);
  for (auto &L : m->layers) {
    if (L.mla) blok_mla_layer_destroy(L.mla);
    if (L.moe) blok_moe_layer_destroy(L.moe);
  }
  cudaError_t first = cudaSuccess;
  for (void *p : m->allocations) {
    cudaError_t e = cudaFree(p);
    if (first == cudaSuccess) first = e;
  }
  delete m;
  return first == cudaSuccess ? BLOK_OK : cuda_fail(first, "cudaFree(model)");
}

extern "C" int blok_model_create_synthetic(const blok_model_config *cfg, uint64_t seed, blok_model_t **out) {
  BLOK_REQUIRE(cfg && out, BLOK_ERR_ARG, "blok_model_create_synthetic: null pointer");
  BLOK_REQUIRE(cfg->layers >= 1 && cfg->first_dense >= 0 && cfg->first_dense <= cfg->layers && cfg->vocab > 0 &&
                   cfg->hidden % 256 == 0 && cfg->max_batch >= 1 && cfg->max_batch <= kMaxBatch && cfg->max_ctx >= 1 &&
                   cfg->prefill_chunk >= 0 && cfg->prefill_chunk <= kMaxBatch,
               BLOK_ERR_SHAPE, "blok_model_create_synthetic: unsupported configuration");
  BLOK_REQUIRE(cfg->kv_page_rows == 0 || (cfg->kv_page_rows >= 32 && cfg->kv_page_rows % 32 == 0 && cfg->kv_pages >= 1),
               BLOK_ERR_SHAPE, "blok_model_create_synthetic: kv_page_rows %d must be 0 or a multiple of 32 with kv_pages >= 1",
               cfg->kv_page_rows);
  BLOK_REQUIRE(cfg->first_dense == 0 || (cfg->dense_inter > 0 && cfg->dense_inter % 32 == 0), BLOK_ERR_SHAPE,
               "blok_model_create_synthetic: dense_inter %d must be a positive multiple of 32", cfg->dense_inter);
  BLOK_REQUIRE(cfg->ep_world <= 1 || (cfg->ep_rank >= 0 && cfg->ep_rank < cfg->ep_world && cfg->experts % cfg->ep_world == 0 &&
                                       cfg->hidden % 512 == 0 && cfg->inter % 512 == 0 && cfg->kv_page_rows == 0),
               BLOK_ERR_SHAPE, "blok_model_create_synthetic: expert parallelism needs 0 <= ep_rank < ep_world, experts divisible "
                               "by ep_world, hidden and inter multiples of 512 and a dense cache");
  blok_model *m = new (std::nothrow) blok_model();
  BLOK_REQUIRE(m, BLOK_ERR_ARG, "blok_model_create_synthetic: out of host memory");
  m->cfg = *cfg;
  // a step's launches are replayed from a CUDA graph, the all-reduces of a sharded model among them (measured on 2 GPUs:
  // 5.7 ms against 6.3 ms per token eagerly); BLOK_MODEL_GRAPH=0 keeps every launch eager
  if (const char *g = getenv("BLOK_MODEL_GRAPH")) m->graphs_enabled = strcmp(g, "0") != 0;
  m->seed = seed;
  int rc = build(m);
  if (rc) {
    blok_model_destroy(m);
    return rc;
  }
  *out = m;
  return BLOK_OK;
}

extern "C" int blok_model_tensor(blok_model_t *m, int layer, const char *name, void **ptr, size_t *bytes) {
  BLOK_REQUIRE(m && name && ptr && bytes, BLOK_ERR_ARG, "blok_model_tensor: null pointer");
  const std::map<std::string, Tensor> *map = nullptr;
  if (layer == -1) map = &m->top;
  else if (layer >= 0 && layer < (int)m->layers.size()) map = &m->layers[layer].t;
  BLOK_REQUIRE(map, BLOK_ERR_ARG, "blok_model_tensor: layer %d out of range", layer);
  auto it = map->find(name);
  BLOK_REQUIRE(it != map->end(), BLOK_ERR_ARG, "blok_model_tensor: layer %d has no tensor '%s'", layer, name);
  *ptr = it->second.ptr;
  *bytes = it->second.bytes;
  return BLOK_OK;
}

extern "C" int blok_model_get_config(blok_model_t *m, blok_model_config *cfg) {
  BLOK_REQUIRE(m && cfg, BLOK_ERR_ARG, "blok_model_get_config: null pointer");
  *cfg = m->cfg;
  return BLOK_OK;
}

extern "C" int blok_model_hidden(blok_model_t *m, const blok_bf16_t **ptr, int *rows) {
  BLOK_REQUIRE(m && ptr && rows, BLOK_ERR_ARG, "blok_model_hidden: null pointer");
  *ptr = m->n;
  *rows = m->rows;
  return BLOK_OK;
}

extern "C" int blok_model_refresh_derived(blok_model_t *m) {
  BLOK_REQUIRE(m, BLOK_ERR_ARG, "blok_model_refresh_derived: null pointer");
  for (auto &L : m->layers)
    if (L.mla)
      if (int rc = blok_mla_layer_refresh(L.mla)) return rc;
  return BLOK_OK;
}

extern "C" int blok_model_set_comm(blok_model_t *m, blok_comm_t *comm) {
  BLOK_REQUIRE(m && comm, BLOK_ERR_ARG, "blok_model_set_comm: null pointer");
  BLOK_REQUIRE(m->cfg.ep_world > 1 && blok_comm_world(comm) == m->cfg.ep_world && blok_comm_rank(comm) == m->cfg.ep_rank, BLOK_ERR_STATE,
               "blok_model_set_comm: the communicator is rank %d of %d, the model was created as rank %d of %d", blok_comm_rank(comm),
               blok_comm_world(comm), m->cfg.ep_rank, m->cfg.ep_world);
  m->comm = comm;
  return BLOK_OK;
}

extern "C" int blok_model_check(blok_model_t *m, blok_stream_t stream) {
  BLOK_REQUIRE(m, BLOK_ERR_ARG, "blok_model_check: null pointer");
  int first = BLOK_OK;
  std::string message;
  for (size_t l = 0; l < m->layers.size(); ++l) {
    auto &L = m->layers[l];
    int rc = L.moe ? blok_moe_layer_check(L.moe, stream) : BLOK_OK;
    if (rc == BLOK_OK && L.mla) rc = blok_mla_layer_check(L.mla, stream);
    if (rc != BLOK_OK && first == BLOK_OK) {  // keep checking: every layer's error word is cleared by its check
      first = rc;
      message = "layer " + std::to_string(l) + ": " + blok_last_error();
    }
  }
  if (first == BLOK_OK && m->comm) return blok_comm_check(m->comm);
  if (first != BLOK_OK) set_error("%s", message.c_str());
  return first;
}

extern "C" int blok_model_debug_set_layer_error(blok_model_t *m, int layer, unsigned code, blok_stream_t stream) {
  BLOK_REQUIRE(m && layer >= 0 && layer < (int)m->layers.size() && m->layers[layer].moe, BLOK_ERR_ARG,
               "blok_model_debug_set_layer_error: layer %d is not a MoE layer of this model", layer);
  return blok_moe_layer_debug_set_error(m->layers[layer].moe, code, stream);
}

extern "C" int blok_model_reset(blok_model_t *m) {
  BLOK_REQUIRE(m, BLOK_ERR_ARG, "blok_model_reset: null pointer");
  BLOK_CUDA(cudaMemset(m->pos, 0, m->cfg.max_batch * 4));
  for (int s = 0; s < m->cfg.max_batch; ++s) {
    m->host_pos[s] = 0;
    if (m->pages) blok_kv_pages_release(m->pages, s);
  }
  return BLOK_OK;
}

// The MoE layer with the experts split over the ranks, for T rows that every rank holds alike (the attention block is
// replicated): route (replicated, so all ranks agree without talking), run the selected experts this rank holds, add the
// ranks' weighted sums with ONE all-reduce, round, add the shared expert (replicated).  m->n -> m->tmp.
static int moe_sharded_rows(blok_model_t *m, blok::LayerWeights &L, int T, blok_stream_t stream_) {
  const blok_model_config &c = m->cfg;
  cudaStream_t stream = (cudaStream_t)stream_;
  BLOK_REQUIRE(m->comm, BLOK_ERR_STATE, "blok_model_step: a model with ep_world > 1 needs blok_model_set_comm first");
  const uint16_t *router = tp<uint16_t>(L.t, "router");
  int rc;
  const dim3 grid((c.hidden / 2 + 255) / 256, T);
  if (T <= 3 && blok_moe_layer_has_partial(L.moe)) {
    // steps of up to three sequences: one launch per row does the router, the shared expert and this rank's selected
    // experts (measured on 2 GPUs, 9 layers: 3.0 ms against 3.6 ms through the grouped kernels at batch 2, 4.5 against 4.0
    // at batch 4)
    for (int b = 0; b < T; ++b)
      if ((rc = blok_moe_decode_partial(L.moe, m->n + (size_t)b * c.hidden, m->ep_part + (size_t)b * c.hidden,
                                        m->ep_shared + (size_t)b * c.hidden, nullptr, nullptr, stream_)))
        return rc;
    if ((rc = blok_comm_all_reduce_f32(m->comm, m->ep_part, (long)T * c.hidden, stream_))) return rc;
    sharded_finish_kernel<<<grid, 256, 0, stream>>>(m->ep_part, m->ep_shared, c.hidden, m->tmp);
    return launch_status("sharded_finish_kernel");
  }
  // router logits (fp32): 9..64 rows in one pass of the weight-streaming kernel where the sizes fit it, else 8 rows at a time
  const bool stream_rows = T > 8 && c.experts % 16 == 0 && c.hidden % 256 == 0;
  for (int t0 = 0; t0 < T; t0 += stream_rows ? kWgStreamTokens : 8) {
    const int nrows = std::min(T - t0, stream_rows ? kWgStreamTokens : 8);
    rc = nrows > 8 ? launch_wgemm_rows(WG_BF16_PLAIN, router, nullptr, m->n + (size_t)t0 * c.hidden, nullptr, m->ep_logits + (size_t)t0 * c.experts,
                                       c.experts, c.hidden, nrows, m->ep_sk, m->ep_sk_bytes, stream)
                   : launch_bf16_gemv(router, m->n + (size_t)t0 * c.hidden, nullptr, m->ep_logits + (size_t)t0 * c.experts, c.experts, c.hidden,
                                      nrows, stream);
    if (rc) return rc;
  }
  if ((rc = launch_router_topk(m->ep_logits, tp<float>(L.t, "router_bias"), T, c.experts, c.topk, c.routed_scale, m->ep_ids, m->ep_wts,
                               m->ep_local_ids, m->ep_base, stream)))
    return rc;
  // assignments of experts held elsewhere carry ids outside [0, ep_local): the grouped kernels skip them
  if ((rc = blok_moe_experts_grouped(L.moe, m->n, m->ep_rows, m->ep_local_ids, T * c.topk, m->ep_y, stream_))) return rc;
  sharded_partial_kernel<<<grid, 256, 0, stream>>>(m->ep_y, m->ep_wts, m->ep_local_ids, m->ep_local, c.hidden, c.topk, m->ep_part);
  if ((rc = launch_status("sharded_partial_kernel"))) return rc;
  if ((rc = blok_comm_all_reduce_f32(m->comm, m->ep_part, (long)T * c.hidden, stream_))) return rc;
  const uint16_t *shared = nullptr;
  if (c.shared_inter > 0) {
    if ((rc = blok_moe_shared(L.moe, m->n, T, m->ep_shared, stream_))) return rc;
    shared = m->ep_shared;
  }
  sharded_finish_kernel<<<grid, 256, 0, stream>>>(m->ep_part, shared, c.hidden, m->tmp);
  return launch_status("sharded_finish_kernel");
}

// The feed-forward half of layer l for T rows: m->n -> m->tmp (:829-877 without the residual add).  Steps of up to 3
// sequences take the batch-1 kernels row by row; prefill chunks and larger steps take the grouped kernels for the routed
// experts where the sizes fit them, and the dense layer up to 64 rows at a time.
static int ffn_rows(blok_model_t *m, int l, int T, bool chunk, blok_stream_t stream_) {
  const blok_model_config &c = m->cfg;
  auto &L = m->layers[l];
  const size_t H = c.hidden;
  // the grouped kernels stream each selected expert once for all rows: from four rows on that is cheaper than a launch
  // of the batch-1 kernel per row (12-layer model, 8 sequences: 10.2 ms a step row by row)
  const bool wide = chunk ? T > 1 : T > 3;
  int rc = BLOK_OK;
  if (l < c.first_dense) {
    // rows per call: up to 8, fewer when 8 rows of the wider of the two vectors would not fit in shared memory
    const size_t row_bytes = (size_t)(c.hidden > c.dense_inter ? c.hidden : c.dense_inter) * 2 + 64;
    int group = wide ? 8 : 1;
    while (group > 1 && row_bytes * group > 200 * 1024) --group;
    if (wide && T > 8 && m->mlp_rows > 8) group = m->mlp_rows;  // one pass over the weights for up to 64 rows
    for (int b = 0; b < T && !rc; b += group)
      rc = blok_bf16_mlp(tp<uint16_t>(L.t, "gate_proj"), tp<uint16_t>(L.t, "up_proj"), tp<uint16_t>(L.t, "down_proj"), m->n + b * H,
                         m->tmp + b * H, c.hidden, c.dense_inter, T - b < group ? T - b : group, m->mlp_ws, m->mlp_ws_bytes, stream_);
    return rc;
  }
  if (c.ep_world > 1) return moe_sharded_rows(m, L, T, stream_);
  if (wide && m->moe_batched_ok) return blok_moe_batched(L.moe, m->n, T, m->tmp, nullptr, nullptr, stream_);
  for (int b = 0; b < T && !rc; ++b) rc = blok_moe_decode(L.moe, m->n + b * H, m->tmp + b * H, nullptr, nullptr, stream_);
  return rc;
}

// Embedding and every layer for T rows of m->ids; leaves the final-normed hidden states in m->n.  chunk: the rows are
// consecutive tokens of sequence 0 (a prefill chunk); otherwise row b is the next token of sequence b.
static int layers_body(blok_model_t *m, int T, bool chunk, blok_stream_t stream_) {
  const blok_model_config &c = m->cfg;
  int rc;
  if ((rc = blok_embed(tp<uint16_t>(m->top, "embed_tokens"), m->ids, c.vocab, c.hidden, T, m->x, stream_))) return rc;  // :802
  // Every residual add is fused with the RMSNorm that follows it (blok_add_rmsnorm), so a layer is: attention on n,
  // x += attention | n = norm(x), feed-forward on n, x += feed-forward | n = the next layer's (or the final) norm.
  if ((rc = blok_rmsnorm(m->x, tp<uint16_t>(m->layers[0].t, "input_layernorm"), m->n, T, c.hidden, c.rms_eps, stream_))) return rc;
  for (int l = 0; l < c.layers; ++l) {
    auto &L = m->layers[l];
    // attention block, :812-827
    if (m->pages)  // entry b is slot slot_of[b] at position ctx_b[b], for steps and chunks alike
      rc = blok_mla_decode_paged(L.mla, m->n, L.cache, m->table_dev, m->slot_of, m->table_stride, c.kv_page_rows, m->ctx_b, T, m->tmp,
                                 stream_);
    else
      rc = chunk ? blok_mla_prefill(L.mla, m->n, L.cache, c.max_ctx, m->pos, T, m->tmp, stream_)
                 : blok_mla_decode(L.mla, m->n, L.cache, c.max_ctx, m->pos, T, m->tmp, stream_);
    if (rc) return rc;
    if ((rc = blok_add_rmsnorm(m->x, m->tmp, tp<uint16_t>(L.t, "post_attention_layernorm"), m->n, T, c.hidden, c.rms_eps, stream_)))
      return rc;
    if ((rc = ffn_rows(m, l, T, chunk, stream_))) return rc;  // :829-877
    const bool last = l + 1 == c.layers;
    const uint16_t *next_ln = last ? tp<uint16_t>(m->top, "norm") : tp<uint16_t>(m->layers[l + 1].t, "input_layernorm");  // :812 / :880
    if ((rc = blok_add_rmsnorm(m->x, m->tmp, next_ln, m->n, T, c.hidden, last ? c.final_rms_eps : c.rms_eps, stream_))) return rc;
  }
  return BLOK_OK;
}

// The launches of one decode step on `stream`, reading m->ids and writing m->next; every position and length is device
// resident, so the same sequence of launches serves every step and can be replayed from a graph.
static int step_body(blok_model_t *m, int B, blok_stream_t stream_) {
  const blok_model_config &c = m->cfg;
  cudaStream_t stream = (cudaStream_t)stream_;
  int rc;
  if ((rc = layers_body(m, B, false, stream_))) return rc;
  // the sampler takes 64 rows per call where the sizes fit the weight-streaming kernel (one pass over the table), else 8
  const int head_rows = (c.vocab % 16 == 0 && c.hidden % 256 == 0) ? kWgStreamTokens : 8;
  for (int b = 0; b < B; b += head_rows)
    if ((rc = blok_lm_head_argmax(tp<uint16_t>(m->top, "lm_head"), m->n + (size_t)b * c.hidden, c.vocab, c.hidden,
                                  B - b < head_rows ? B - b : head_rows, m->next + b, m->head_ws, m->head_ws_bytes, stream_)))
      return rc;
  if (m->pages) advance_slots_kernel<<<1, 64, 0, stream>>>(m->pos, m->slot_of, B);
  else advance_kernel<<<1, 64, 0, stream>>>(m->pos, B, 1);
  return launch_status("advance_kernel");
}

extern "C" int blok_model_step_slots(blok_model_t *m, const int *slots, int B, const uint32_t *ids, uint32_t *next_ids,
                                     blok_stream_t stream_) {
  BLOK_REQUIRE(m && slots && ids && next_ids, BLOK_ERR_ARG, "blok_model_step_slots: null pointer");
  const blok_model_config &c = m->cfg;
  BLOK_REQUIRE(B >= 1 && B <= c.max_batch, BLOK_ERR_SHAPE, "blok_model_step_slots: B=%d outside [1, %d]", B, c.max_batch);
  bool identity = true;
  for (int b = 0; b < B; ++b) {
    BLOK_REQUIRE(slots[b] >= 0 && slots[b] < c.max_batch, BLOK_ERR_ARG, "blok_model_step_slots: slot %d outside [0, %d)", slots[b],
                 c.max_batch);
    for (int a = 0; a < b; ++a) BLOK_REQUIRE(slots[a] != slots[b], BLOK_ERR_ARG, "blok_model_step_slots: slot %d named twice", slots[b]);
    BLOK_REQUIRE(m->host_pos[slots[b]] + 1 <= c.max_ctx, BLOK_ERR_SHAPE,
                 "blok_model_step_slots: the sequence in slot %d already holds max_ctx = %d tokens", slots[b], c.max_ctx);  // :205
    identity = identity && slots[b] == b;
  }
  if (!m->pages) {
    BLOK_REQUIRE(identity, BLOK_ERR_STATE, "blok_model_step_slots: a model with a dense cache steps slots 0..B-1 only");
    return blok_model_step(m, ids, B, next_ids, stream_);
  }
  cudaStream_t stream = (cudaStream_t)stream_;
  int rc;
  for (int b = 0; b < B; ++b)
    if ((rc = blok_kv_pages_reserve(m->pages, slots[b], m->host_pos[slots[b]] + 1))) return rc;
  if ((rc = blok_kv_pages_upload(m->pages, m->table_dev, stream_))) return rc;
  BLOK_CUDA(cudaMemcpyAsync(m->slot_of, slots, (size_t)B * 4, cudaMemcpyHostToDevice, stream));
  if (ids != m->ids) BLOK_CUDA(cudaMemcpyAsync(m->ids, ids, (size_t)B * 4, cudaMemcpyDeviceToDevice, stream));
  gather_positions_kernel<<<1, 64, 0, stream>>>(m->pos, m->slot_of, B, m->ctx_b);
  if ((rc = launch_status("gather_positions_kernel"))) return rc;
  if ((rc = step_body(m, B, stream_))) return rc;
  for (int b = 0; b < B; ++b) ++m->host_pos[slots[b]];
  if (next_ids != m->next) BLOK_CUDA(cudaMemcpyAsync(next_ids, m->next, (size_t)B * 4, cudaMemcpyDeviceToDevice, stream));
  return BLOK_OK;
}

extern "C" int blok_model_step(blok_model_t *m, const uint32_t *ids, int B, uint32_t *next_ids, blok_stream_t stream_) {
  BLOK_REQUIRE(m && ids && next_ids, BLOK_ERR_ARG, "blok_model_step: null pointer");
  BLOK_REQUIRE(B >= 1 && B <= m->cfg.max_batch, BLOK_ERR_SHAPE, "blok_model_step: B=%d outside [1, %d]", B, m->cfg.max_batch);
  if (m->pages) {
    int slots[kMaxBatch];
    for (int b = 0; b < B; ++b) slots[b] = b;
    return blok_model_step_slots(m, slots, B, ids, next_ids, stream_);
  }
  for (int b = 0; b < B; ++b)
    BLOK_REQUIRE(m->host_pos[b] + 1 <= m->cfg.max_ctx, BLOK_ERR_SHAPE, "blok_model_step: sequence %d already holds max_ctx = %d tokens", b,
                 m->cfg.max_ctx);  // the reference's capacity check, :205
  for (int b = 0; b < B; ++b) ++m->host_pos[b];
  cudaStream_t stream = (cudaStream_t)stream_;
  if (ids != m->ids) BLOK_CUDA(cudaMemcpyAsync(m->ids, ids, (size_t)B * 4, cudaMemcpyDeviceToDevice, stream));
  int rc = BLOK_OK;
  // The first step of a batch size runs eagerly, the second is captured (nothing executes during capture) and
  // replayed at once, later steps replay the graph.  The legacy default stream cannot be captured.
  const bool can_graph = m->graphs_enabled && stream != nullptr && stream != cudaStreamLegacy;
  if (can_graph && m->step_graph[B]) {
    BLOK_CUDA(cudaGraphLaunch(m->step_graph[B], stream));
    count_launches(m->graph_launches[B]);
  } else if (can_graph && m->steps_seen[B] >= 1) {
    cudaGraph_t graph = nullptr;
    cudaError_t e = cudaStreamBeginCapture(stream, cudaStreamCaptureModeThreadLocal);
    if (e == cudaSuccess) {
      const long long before = launches_so_far();
      rc = step_body(m, B, stream_);
      m->graph_launches[B] = launches_so_far() - before;
      count_launches(-m->graph_launches[B]);  // nothing ran during the capture
      cudaError_t e2 = cudaStreamEndCapture(stream, &graph);
      if (rc == BLOK_OK && e2 == cudaSuccess && graph) e = cudaGraphInstantiate(&m->step_graph[B], graph, 0);
      else e = e2 == cudaSuccess ? cudaErrorUnknown : e2;
      if (graph) cudaGraphDestroy(graph);
    }
    if (e != cudaSuccess || !m->step_graph[B]) {  // capture is not possible here: stay with eager launches
      cudaGetLastError();
      m->step_graph[B] = nullptr;
      m->graphs_enabled = false;
      rc = step_body(m, B, stream_);
    } else {
      BLOK_CUDA(cudaGraphLaunch(m->step_graph[B], stream));
      count_launches(m->graph_launches[B]);
      rc = BLOK_OK;
    }
  } else {
    rc = step_body(m, B, stream_);
    ++m->steps_seen[B];
  }
  if (rc) return rc;
  if (next_ids != m->next) BLOK_CUDA(cudaMemcpyAsync(next_ids, m->next, (size_t)B * 4, cudaMemcpyDeviceToDevice, stream));
  return BLOK_OK;
}

extern "C" int blok_model_prefill_slot(blok_model_t *m, int slot, const uint32_t *ids, int n, uint32_t *next_id, blok_stream_t stream_) {
  BLOK_REQUIRE(m && ids && next_id, BLOK_ERR_ARG, "blok_model_prefill: null pointer");
  BLOK_REQUIRE(m->cfg.prefill_chunk >= 1, BLOK_ERR_STATE, "blok_model_prefill: the model was created with prefill_chunk = 0");
  BLOK_REQUIRE(n >= 1, BLOK_ERR_ARG, "blok_model_prefill: no tokens");
  const blok_model_config &c = m->cfg;
  BLOK_REQUIRE(slot >= 0 && slot < c.max_batch && (m->pages || slot == 0), BLOK_ERR_ARG,
               "blok_model_prefill: slot %d (a model with a dense cache prefills sequence 0 only)", slot);
  BLOK_REQUIRE(m->host_pos[slot] + n <= c.max_ctx, BLOK_ERR_SHAPE, "blok_model_prefill: %ld cached + %d new tokens exceed max_ctx = %d",
               m->host_pos[slot], n, c.max_ctx);  // :205
  cudaStream_t stream = (cudaStream_t)stream_;
  int rc;
  if (m->pages && (rc = blok_kv_pages_reserve(m->pages, slot, m->host_pos[slot] + n))) return rc;  // all or nothing, before any launch
  if (m->pages && (rc = blok_kv_pages_upload(m->pages, m->table_dev, stream_))) return rc;
  for (int at = 0; at < n; at += c.prefill_chunk) {
    const int T = n - at < c.prefill_chunk ? n - at : c.prefill_chunk;
    BLOK_CUDA(cudaMemcpyAsync(m->ids, ids + at, (size_t)T * 4, cudaMemcpyDeviceToDevice, stream));
    if (m->pages) {
      chunk_slots_kernel<<<1, 64, 0, stream>>>(m->pos, slot, T, m->ctx_b, m->slot_of);
      if ((rc = launch_status("chunk_slots_kernel"))) return rc;
    }
    if ((rc = layers_body(m, T, true, stream_))) return rc;
    if (at + T == n) {  // only the prompt's last token is sampled (:886 keeps the last step's id)
      if ((rc = blok_lm_head_argmax(tp<uint16_t>(m->top, "lm_head"), m->n + (size_t)(T - 1) * c.hidden, c.vocab, c.hidden, 1, m->next,
                                    m->head_ws, m->head_ws_bytes, stream_)))
        return rc;
    }
    advance_kernel<<<1, 64, 0, stream>>>(m->pos + slot, 1, T);
    if ((rc = launch_status("advance_kernel"))) return rc;
    m->host_pos[slot] += T;
  }
  if (next_id != m->next) BLOK_CUDA(cudaMemcpyAsync(next_id, m->next, 4, cudaMemcpyDeviceToDevice, stream));
  return BLOK_OK;
}

extern "C" int blok_model_prefill(blok_model_t *m, const uint32_t *ids, int n, uint32_t *next_id, blok_stream_t stream) {
  return blok_model_prefill_slot(m, 0, ids, n, next_id, stream);
}

extern "C" int blok_model_slot_release(blok_model_t *m, int slot, blok_stream_t stream) {
  BLOK_REQUIRE(m, BLOK_ERR_ARG, "blok_model_slot_release: null pointer");
  BLOK_REQUIRE(slot >= 0 && slot < m->cfg.max_batch, BLOK_ERR_ARG, "blok_model_slot_release: slot %d outside [0, %d)", slot,
               m->cfg.max_batch);
  BLOK_CUDA(cudaMemsetAsync(m->pos + slot, 0, 4, (cudaStream_t)stream));
  m->host_pos[slot] = 0;
  return m->pages ? blok_kv_pages_release(m->pages, slot) : BLOK_OK;
}

extern "C" long blok_model_slot_length(blok_model_t *m, int slot) {
  return (m && slot >= 0 && slot < m->cfg.max_batch) ? m->host_pos[slot] : -1;
}

extern "C" int blok_model_free_pages(blok_model_t *m) { return (m && m->pages) ? blok_kv_pages_free_count(m->pages) : -1; }

extern "C" int blok_model_generate(blok_model_t *m, const uint32_t *prompt, int n_prompt, int max_new, uint32_t *out,
                                   int *n_out) {
  BLOK_REQUIRE(m && prompt && out && n_out, BLOK_ERR_ARG, "blok_model_generate: null pointer");
  BLOK_REQUIRE(n_prompt >= 1 && max_new >= 1, BLOK_ERR_ARG, "blok_model_generate: empty prompt or max_new < 1");
  BLOK_REQUIRE((long)n_prompt + max_new <= m->cfg.max_ctx, BLOK_ERR_SHAPE,
               "blok_model_generate: requested sequence exceeds the model's context (%d)", m->cfg.max_ctx);  // :784
  for (int i = 0; i < n_prompt; ++i)
    BLOK_REQUIRE(prompt[i] < (uint32_t)m->cfg.vocab, BLOK_ERR_ARG, "blok_model_generate: prompt token outside vocabulary");
  int rc = blok_model_reset(m);
  if (rc) return rc;
  *n_out = 0;
  uint32_t next = prompt[0];
  if (m->cfg.prefill_chunk >= 1) {
    // the prompt in chunks: every layer's weights are read once per chunk instead of once per token
    BLOK_CUDA(cudaMemcpyAsync(m->prompt_ids, prompt, (size_t)n_prompt * 4, cudaMemcpyHostToDevice, nullptr));
    if ((rc = blok_model_prefill(m, m->prompt_ids, n_prompt, m->next, nullptr))) return rc;
  } else {
    // prompt replay, token by token; only the last step's sample is used (:886)
    for (int i = 0; i < n_prompt; ++i) {
      BLOK_CUDA(cudaMemcpyAsync(m->ids, prompt + i, 4, cudaMemcpyHostToDevice, nullptr));
      if ((rc = blok_model_step(m, m->ids, 1, m->next, nullptr))) return rc;
    }
  }
  BLOK_CUDA(cudaMemcpy(&next, m->next, 4, cudaMemcpyDeviceToHost));
  for (int i = 0; i < max_new && next != m->cfg.eos_id; ++i) {  // :887-890
    out[(*n_out)++] = next;
    if (i + 1 < max_new) {
      if ((rc = blok_model_step(m, m->next, 1, m->next, nullptr))) return rc;
      BLOK_CUDA(cudaMemcpy(&next, m->next, 4, cudaMemcpyDeviceToHost));
    }
  }
  // a bounded device-side wait that gave up (or a position outside a cache) in any layer makes the tokens void
  return blok_model_check(m, nullptr);
}

// The serving loop of blok_model_generate_many over an existing batcher (the caller destroys it).
static int serve_requests(blok_model_t *m, blok_batcher_t *bt, const uint32_t *prompts, const int *prompt_offsets, int n_requests,
                          int max_new, uint32_t *out, int *n_out) {
  const blok_model_config &c = m->cfg;
  int rc = BLOK_OK;
  for (int r = 0; r < n_requests && !rc; ++r) {
    int id = -1;
    rc = blok_batcher_submit(bt, prompt_offsets[r + 1] - prompt_offsets[r], max_new, &id);
    n_out[r] = 0;
  }
  std::vector<int> admit_slots(c.max_batch), admit_req(c.max_batch), decode_slots(c.max_batch), slot_req(c.max_batch, -1);
  std::vector<uint32_t> last(c.max_batch, 0), ids(c.max_batch), sampled(c.max_batch);
  // one sampled token of the sequence in `slot`: emitted unless it is EOS (:887); the batcher says whether the sequence ended
  auto take = [&](int slot, uint32_t tok) -> int {
    const int r = slot_req[slot];
    const int eos = tok == c.eos_id;
    if (!eos) out[(size_t)r * max_new + n_out[r]++] = tok;
    last[slot] = tok;
    int finished = 0;
    int e = blok_batcher_token(bt, slot, eos, &finished);
    if (e) return e;
    if (finished) {
      slot_req[slot] = -1;
      return blok_model_slot_release(m, slot, nullptr);
    }
    return BLOK_OK;
  };
  while (!rc && blok_batcher_unfinished(bt) > 0) {
    int n_admit = 0, n_decode = 0;
    if ((rc = blok_batcher_plan(bt, admit_slots.data(), admit_req.data(), &n_admit, decode_slots.data(), &n_decode))) break;
    if (n_admit == 0 && n_decode == 0) {  // cannot happen: submit refused what can never fit, and finished sequences free their budget
      set_error("blok_model_generate_many: no sequence can make progress");
      rc = BLOK_ERR_STATE;
      break;
    }
    if (n_decode) {  // the running sequences step together; their ids come back for the EOS test, as at :882
      for (int b = 0; b < n_decode; ++b) ids[b] = last[decode_slots[b]];
      BLOK_CUDA(cudaMemcpyAsync(m->prompt_ids, ids.data(), (size_t)n_decode * 4, cudaMemcpyHostToDevice, nullptr));
      if ((rc = blok_model_step_slots(m, decode_slots.data(), n_decode, m->prompt_ids, m->next, nullptr))) break;
      BLOK_CUDA(cudaMemcpy(sampled.data(), m->next, (size_t)n_decode * 4, cudaMemcpyDeviceToHost));
      for (int b = 0; b < n_decode && !rc; ++b) rc = take(decode_slots[b], sampled[b]);
      if (rc) break;
    }
    for (int a = 0; a < n_admit && !rc; ++a) {  // arrivals: the prompt in chunks, its last token sampled
      const int slot = admit_slots[a], r = admit_req[a];
      const int n = prompt_offsets[r + 1] - prompt_offsets[r];
      slot_req[slot] = r;
      BLOK_CUDA(cudaMemcpyAsync(m->prompt_ids, prompts + prompt_offsets[r], (size_t)n * 4, cudaMemcpyHostToDevice, nullptr));
      if ((rc = blok_model_prefill_slot(m, slot, m->prompt_ids, n, m->next, nullptr))) break;
      uint32_t tok = 0;
      BLOK_CUDA(cudaMemcpy(&tok, m->next, 4, cudaMemcpyDeviceToHost));
      rc = take(slot, tok);
    }
  }
  return rc;
}

extern "C" int blok_model_generate_many(blok_model_t *m, const uint32_t *prompts, const int *prompt_offsets, int n_requests,
                                        int max_new, uint32_t *out, int *n_out) {
  BLOK_REQUIRE(m && prompts && prompt_offsets && out && n_out, BLOK_ERR_ARG, "blok_model_generate_many: null pointer");
  BLOK_REQUIRE(m->pages && m->cfg.prefill_chunk >= 1, BLOK_ERR_STATE,
               "blok_model_generate_many: needs a paged model (kv_page_rows > 0) with prefill_chunk >= 1");
  BLOK_REQUIRE(n_requests >= 1 && max_new >= 1, BLOK_ERR_ARG, "blok_model_generate_many: no requests or max_new < 1");
  const blok_model_config &c = m->cfg;
  for (int r = 0; r < n_requests; ++r) {
    BLOK_REQUIRE(prompt_offsets[r + 1] > prompt_offsets[r], BLOK_ERR_ARG, "blok_model_generate_many: request %d has an empty prompt", r);
    for (int i = prompt_offsets[r]; i < prompt_offsets[r + 1]; ++i)
      BLOK_REQUIRE(prompts[i] < (uint32_t)c.vocab, BLOK_ERR_ARG, "blok_model_generate_many: prompt token outside vocabulary");  // :552
  }
  int rc = blok_model_reset(m);
  if (rc) return rc;
  blok_batcher_t *bt = nullptr;
  if ((rc = blok_batcher_create(c.max_batch, c.kv_pages, c.kv_page_rows, c.max_ctx, &bt))) return rc;
  rc = serve_requests(m, bt, prompts, prompt_offsets, n_requests, max_new, out, n_out);
  blok_batcher_destroy(bt);
  return rc ? rc : blok_model_check(m, nullptr);
}
