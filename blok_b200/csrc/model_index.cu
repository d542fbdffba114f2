// Runtime-index loader: brings a materialised checkpoint into a model handle's resident
// tensors.  Mirrors the behaviour of the reference's index reader and forward contract
// (runtime_index src/kimi_exec.cu:559-581, need / bf16 / validate_i4_pair :583-606,
// validate_forward_contract :736-778; the index is written by scripts/model_fetch.py:113-127)
// with the shapes taken from the model's configuration instead of compile-time constants,
// so that a tiny index written by a test exercises the same checks.
//
// The reference reads every tensor again for every token through its storage layer; here
// each tensor is read once with pread, staged through pinned memory and copied into the
// model's HBM-resident tensor (routed experts into their slice of the expert-major arrays).
#include <fcntl.h>
#include <unistd.h>

#include <cerrno>
#include <cstring>
#include <fstream>
#include <map>
#include <sstream>
#include <string>
#include <vector>

#include "common.cuh"

namespace blok {
namespace {

struct IndexTensor {
  std::string name, role, slot, dtype, shape, file;
  int layer = -1, expert = -1;
  unsigned long long off = 0, bytes = 0, align = 0, data = 0, data_bytes = 0;
};

struct Index {
  std::map<std::string, IndexTensor> tensors;  // "layer:expert:role:slot"
};

std::string key_of(int layer, int expert, const std::string &role, const std::string &slot) {
  return std::to_string(layer) + ":" + std::to_string(expert) + ":" + role + ":" + slot;
}

bool parse_int(const std::string &s, int *out) {
  if (s.empty()) return false;
  char *end = nullptr;
  errno = 0;
  long v = strtol(s.c_str(), &end, 10);
  if (errno || *end || v < -1 || v > 1 << 30) return false;
  *out = (int)v;
  return true;
}

// Reads and checks the text index: header line, then one "tensor" line of 14 fields per tensor.
int read_index(const char *path, Index *out) {
  std::ifstream in(path);
  BLOK_REQUIRE(in.good(), BLOK_ERR_ARG, "runtime index: cannot open %s", path);
  std::string line;
  BLOK_REQUIRE(std::getline(in, line) && line == "blok-runtime-index-v1", BLOK_ERR_ARG, "runtime index: bad header in %s", path);
  int lineno = 1;
  while (std::getline(in, line)) {
    ++lineno;
    BLOK_REQUIRE(line.rfind("tensor ", 0) == 0, BLOK_ERR_ARG, "runtime index: line %d is not a tensor line", lineno);
    std::istringstream ss(line);
    std::string tag, layer, expert, extra;
    IndexTensor t;
    const bool ok = (bool)(ss >> tag >> t.name >> t.role >> layer >> expert >> t.slot >> t.dtype >> t.shape >> t.off >> t.bytes >>
                           t.align >> t.data >> t.data_bytes >> t.file);
    BLOK_REQUIRE(ok, BLOK_ERR_ARG, "runtime index: line %d is incomplete (14 fields expected)", lineno);
    BLOK_REQUIRE(!(ss >> extra), BLOK_ERR_ARG, "runtime index: line %d has trailing fields (paths cannot contain whitespace)", lineno);
    BLOK_REQUIRE(parse_int(layer, &t.layer) && parse_int(expert, &t.expert), BLOK_ERR_ARG,
                 "runtime index: line %d has a bad layer or expert number", lineno);
    const std::string key = key_of(t.layer, t.expert, t.role, t.slot);
    BLOK_REQUIRE(out->tensors.emplace(key, t).second, BLOK_ERR_ARG, "runtime index: duplicate tensor key %s", key.c_str());
  }
  BLOK_REQUIRE(!out->tensors.empty(), BLOK_ERR_ARG, "runtime index: %s lists no tensors", path);
  return BLOK_OK;
}

int need(const Index &ix, int layer, const char *role, const char *slot, int expert, const IndexTensor **out) {
  const std::string key = key_of(layer, expert, role, slot);
  auto it = ix.tensors.find(key);
  BLOK_REQUIRE(it != ix.tensors.end(), BLOK_ERR_ARG, "runtime index: missing tensor %s", key.c_str());
  *out = &it->second;
  return BLOK_OK;
}

std::string shape_str(long rows, long cols) { return std::to_string(rows) + (cols ? "x" + std::to_string(cols) : ""); }

int need_typed(const Index &ix, int layer, const char *role, const char *slot, int expert, const char *dtype, long rows, long cols,
               size_t elem, const IndexTensor **out) {
  if (int rc = need(ix, layer, role, slot, expert, out)) return rc;
  const IndexTensor &t = **out;
  const unsigned long long bytes = (unsigned long long)rows * (cols ? cols : 1) * elem;
  BLOK_REQUIRE(t.dtype == dtype && t.shape == shape_str(rows, cols) && t.data_bytes == bytes, BLOK_ERR_SHAPE,
               "runtime index: tensor %s is %s %s (%llu bytes), the model needs %s %s (%llu bytes)", t.name.c_str(), t.dtype.c_str(),
               t.shape.c_str(), t.data_bytes, dtype, shape_str(rows, cols).c_str(), bytes);
  return BLOK_OK;
}

// One entry of the load plan: where the tensor's bytes go.
struct Placement {
  const IndexTensor *t;
  int layer;              // model layer, -1 for the top-level tensors
  const char *model_name; // name understood by blok_model_tensor
  int expert;             // >= 0: slice `expert` of an expert-major array
  bool widen_bf16_to_f32; // the router's correction bias is bf16 in the checkpoint and fp32 in the model
};

// The forward contract: every tensor the decode step needs exists with the expected type, shape and byte count,
// and every extent is a sane 4 KiB-aligned read.  Fills the load plan.
int check_contract(const Index &ix, const blok_model_config &c, std::vector<Placement> *plan) {
  for (const auto &kv : ix.tensors) {
    const IndexTensor &t = kv.second;
    BLOK_REQUIRE(!t.slot.empty() && !t.dtype.empty() && !t.shape.empty(), BLOK_ERR_ARG, "runtime index: incomplete metadata for %s",
                 t.name.c_str());
    BLOK_REQUIRE(t.layer < c.layers && t.expert < c.experts, BLOK_ERR_SHAPE, "runtime index: %s is outside the model (layer %d, expert %d)",
                 t.name.c_str(), t.layer, t.expert);
    BLOK_REQUIRE(t.align == 4096 && t.off % t.align == 0 && t.bytes % t.align == 0 && t.data >= t.off && t.data_bytes <= t.bytes &&
                     t.data - t.off <= t.bytes - t.data_bytes,
                 BLOK_ERR_ARG, "runtime index: invalid extent for %s", t.name.c_str());
  }
  const long H = c.hidden, kdim = (long)c.heads * (c.qk_nope + c.qk_rope), vdim = (long)c.heads * c.v_head;
  const IndexTensor *t;
  int rc;
  auto bf = [&](int layer, const char *role, const char *slot, long rows, long cols, const char *model_name) -> int {
    if ((rc = need_typed(ix, layer, role, slot, -1, "bf16", rows, cols, 2, &t))) return rc;
    plan->push_back({t, layer, model_name, -1, false});
    return BLOK_OK;
  };
  for (int i = 0; i < c.layers; ++i) {
    if ((rc = bf(i, "attention_resident", "q_a_proj", c.q_rank, H, "q_a_proj"))) return rc;
    if ((rc = bf(i, "attention_resident", "q_a_layernorm", c.q_rank, 0, "q_a_layernorm"))) return rc;
    if ((rc = bf(i, "attention_resident", "q_b_proj", kdim, c.q_rank, "q_b_proj"))) return rc;
    if ((rc = bf(i, "attention_resident", "kv_a_proj_with_mqa", c.kv_rank + c.qk_rope, H, "kv_a_proj_with_mqa"))) return rc;
    if ((rc = bf(i, "attention_resident", "kv_a_layernorm", c.kv_rank, 0, "kv_a_layernorm"))) return rc;
    if ((rc = bf(i, "attention_resident", "kv_b_proj", (long)c.heads * (c.qk_nope + c.v_head), c.kv_rank, "kv_b_proj"))) return rc;
    if ((rc = bf(i, "attention_resident", "o_proj", H, vdim, "o_proj"))) return rc;
    if ((rc = bf(i, "resident", "input_layernorm", H, 0, "input_layernorm"))) return rc;
    if ((rc = bf(i, "resident", "post_attention_layernorm", H, 0, "post_attention_layernorm"))) return rc;
    if (i < c.first_dense) {
      if ((rc = bf(i, "dense_ffn_rowcol", "gate_proj", c.dense_inter, H, "gate_proj"))) return rc;
      if ((rc = bf(i, "dense_ffn_rowcol", "up_proj", c.dense_inter, H, "up_proj"))) return rc;
      if ((rc = bf(i, "dense_ffn_rowcol", "down_proj", H, c.dense_inter, "down_proj"))) return rc;
      continue;
    }
    if ((rc = bf(i, "router", "gate", c.experts, H, "router"))) return rc;
    if ((rc = need_typed(ix, i, "router", "e_score_correction_bias", -1, "bf16", c.experts, 0, 2, &t))) return rc;
    plan->push_back({t, i, "router_bias", -1, true});
    if (c.shared_inter > 0) {
      if ((rc = bf(i, "shared_expert_resident", "gate_proj", c.shared_inter, H, "shared_gate"))) return rc;
      if ((rc = bf(i, "shared_expert_resident", "up_proj", c.shared_inter, H, "shared_up"))) return rc;
      if ((rc = bf(i, "shared_expert_resident", "down_proj", H, c.shared_inter, "shared_down"))) return rc;
    }
    struct {
      const char *proj, *w_name, *s_name;
      long rows, cols;
    } const projs[3] = {{"gate_proj", "gate_w", "gate_s", c.inter, H}, {"up_proj", "up_w", "up_s", c.inter, H}, {"down_proj", "down_w", "down_s", H, c.inter}};
    for (int e = 0; e < c.experts; ++e) {
      for (const auto &p : projs) {
        const std::string ws = std::string(p.proj) + ".weight_packed", ss = std::string(p.proj) + ".weight_scale";
        if ((rc = need_typed(ix, i, "routed_expert", ws.c_str(), e, "i32", p.rows, p.cols / 8, 4, &t))) return rc;
        plan->push_back({t, i, p.w_name, e, false});
        if ((rc = need_typed(ix, i, "routed_expert", ss.c_str(), e, "bf16", p.rows, p.cols / 32, 2, &t))) return rc;
        plan->push_back({t, i, p.s_name, e, false});
      }
    }
  }
  if ((rc = bf(-1, "resident", "embed_tokens", c.vocab, H, "embed_tokens"))) return rc;
  if ((rc = bf(-1, "resident", "norm", H, 0, "norm"))) return rc;
  if ((rc = bf(-1, "resident", "lm_head", c.vocab, H, "lm_head"))) return rc;
  return BLOK_OK;
}

}  // namespace
}  // namespace blok

using namespace blok;

extern "C" int blok_index_validate(const char *index_path, const blok_model_config *cfg, long *n_tensors, unsigned long long *n_bytes) {
  BLOK_REQUIRE(index_path && cfg, BLOK_ERR_ARG, "blok_index_validate: null pointer");
  Index ix;
  if (int rc = read_index(index_path, &ix)) return rc;
  std::vector<Placement> plan;
  if (int rc = check_contract(ix, *cfg, &plan)) return rc;
  unsigned long long total = 0;
  for (const auto &p : plan) total += p.t->data_bytes;
  if (n_tensors) *n_tensors = (long)plan.size();
  if (n_bytes) *n_bytes = total;
  return BLOK_OK;
}

extern "C" int blok_model_load_index(blok_model_t *model, const char *index_path) {
  BLOK_REQUIRE(model && index_path, BLOK_ERR_ARG, "blok_model_load_index: null pointer");
  blok_model_config cfg;
  if (int rc = blok_model_get_config(model, &cfg)) return rc;
  Index ix;
  if (int rc = read_index(index_path, &ix)) return rc;
  std::vector<Placement> plan;
  if (int rc = check_contract(ix, cfg, &plan)) return rc;

  constexpr size_t kStage = 32u << 20;
  unsigned char *stage = nullptr;
  BLOK_CUDA(cudaMallocHost(&stage, kStage));
  std::map<std::string, int> fds;
  int rc = BLOK_OK;
  std::vector<float> widened;
  for (const auto &p : plan) {
    void *dst = nullptr;
    size_t dst_bytes = 0;
    if ((rc = blok_model_tensor(model, p.layer, p.model_name, &dst, &dst_bytes))) break;
    size_t slice = dst_bytes, at = 0;
    if (p.expert >= 0) {
      // an expert-parallel rank holds experts [base, base + local) only: it reads those and skips the rest
      const int world = cfg.ep_world > 1 ? cfg.ep_world : 1;
      const int local = cfg.experts / world, base = (world > 1 ? cfg.ep_rank : 0) * local;
      if (p.expert < base || p.expert >= base + local) continue;
      slice = dst_bytes / local;
      at = slice * (size_t)(p.expert - base);
    }
    const size_t want = p.widen_bf16_to_f32 ? slice / 2 : slice;
    if (p.t->data_bytes != want) {
      set_error("blok_model_load_index: %s has %llu bytes, the model tensor '%s' takes %zu", p.t->name.c_str(), p.t->data_bytes,
                p.model_name, want);
      rc = BLOK_ERR_SHAPE;
      break;
    }
    auto fd_it = fds.find(p.t->file);
    if (fd_it == fds.end()) {
      const int fd = open(p.t->file.c_str(), O_RDONLY);
      if (fd < 0) {
        set_error("blok_model_load_index: cannot open %s: %s", p.t->file.c_str(), strerror(errno));
        rc = BLOK_ERR_ARG;
        break;
      }
      fd_it = fds.emplace(p.t->file, fd).first;
    }
    for (size_t done = 0; done < p.t->data_bytes && rc == BLOK_OK;) {
      const size_t n = std::min(kStage, (size_t)p.t->data_bytes - done);
      const ssize_t got = pread(fd_it->second, stage, n, (off_t)(p.t->data + done));
      if (got != (ssize_t)n) {
        set_error("blok_model_load_index: short read of %s from %s", p.t->name.c_str(), p.t->file.c_str());
        rc = BLOK_ERR_ARG;
        break;
      }
      cudaError_t ce;
      if (p.widen_bf16_to_f32) {
        widened.resize(n / 2);
        const uint16_t *h = reinterpret_cast<const uint16_t *>(stage);
        for (size_t i = 0; i < n / 2; ++i) {
          const uint32_t bits = (uint32_t)h[i] << 16;
          memcpy(&widened[i], &bits, 4);
        }
        ce = cudaMemcpy(static_cast<unsigned char *>(dst) + at + done * 2, widened.data(), n * 2, cudaMemcpyHostToDevice);
      } else {
        ce = cudaMemcpy(static_cast<unsigned char *>(dst) + at + done, stage, n, cudaMemcpyHostToDevice);
      }
      if (ce != cudaSuccess) {
        set_error("blok_model_load_index: cudaMemcpy: %s", cudaGetErrorString(ce));
        rc = BLOK_ERR_CUDA;
        break;
      }
      done += n;
    }
    if (rc) break;
  }
  for (auto &kv : fds) close(kv.second);
  cudaFreeHost(stage);
  if (rc) return rc;
  // tensors derived from the weights at creation (the transposed W_UK copies) must follow the new weights
  return blok_model_refresh_derived(model);
}
