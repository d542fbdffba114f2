// CPU oracle for the Blok hot path (test infrastructure, NOT a product path).
//
// This file restates, on the host, the arithmetic of the reference executor
// src/kimi_exec.cu for the routed-expert MoE layer and the MLA attention that
// feeds it.  Only tests, the smoke check and the CPU-baseline leg of the bench
// may load it; the CUDA library never links or calls it.
//
// Two evaluation modes:
//   ORC_WIDE (0)      "fp32 evaluation of the reference math": dequantised
//                     weights are rounded to bf16 exactly as the reference does
//                     (src/kimi_exec.cu:312), inputs are bf16 values, every
//                     intermediate stays unrounded (accumulated in fp64) and
//                     only the stated outputs are rounded.  This is the target
//                     the floating-point tolerance is judged against.
//   ORC_REF_EXACT (1) every bf() rounding point of the reference is kept, and
//                     reductions use the reference's schedule: 256 strided
//                     partial sums with fused multiply-add, then a binary tree
//                     (src/kimi_exec.cu:276-282, :305-321).
//
// Parity pin: the reference ships no golden vectors for this path.  The pin is
// (a) the compressed-tensors pack_quantized helpers for the nibble layout,
// (b) the reference's own kernels compiled from their source and launched on a
// GPU through oracle/ref_shim.cu, compared with ORC_REF_EXACT.
//
// Build: see oracle/build.py (g++ -O2 -fopenmp -ffp-contract=off -shared).
#include <cmath>
#include <cstdint>
#include <cstring>
#include <limits>
#include <vector>
#include <algorithm>

#ifdef _OPENMP
#include <omp.h>
#endif

namespace {

constexpr int kGroup = 32;      // src/kimi_exec.cu:181 I4_GROUP
constexpr int kPerWord = 8;     // src/kimi_exec.cu:181 I4_PER_WORD
constexpr int kRefThreads = 256;

inline float bf16_to_f32(uint16_t h) {
  uint32_t u = static_cast<uint32_t>(h) << 16;
  float f;
  std::memcpy(&f, &u, 4);
  return f;
}

// round-to-nearest-even float -> bf16, the same as __float2bfloat16_rn
// (src/kimi_exec.cu:241).
inline uint16_t f32_to_bf16(float f) {
  uint32_t u;
  std::memcpy(&u, &f, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return 0x7fff;  // NaN
  uint32_t lsb = (u >> 16) & 1u;
  u += 0x7fffu + lsb;
  return static_cast<uint16_t>(u >> 16);
}

inline float bf(float v) { return bf16_to_f32(f32_to_bf16(v)); }

// Reference block reduction: s[tid] partials, then for d = 128..1: s[t] += s[t+d].
inline float tree_sum(float *s) {
  for (int d = kRefThreads / 2; d; d >>= 1)
    for (int t = 0; t < d; ++t) s[t] += s[t + d];
  return s[0];
}

inline int nibble_q(uint32_t word, int lane) {  // src/kimi_exec.cu:311
  return static_cast<int>((word >> (4 * lane)) & 0xfu) - 8;
}

// One row of the INT4 mat-vec.  src/kimi_exec.cu:300-323.
float i4_row(const uint32_t *w, const uint16_t *scale, const float *x, int cols, int mode) {
  const int groups = cols / kGroup;
  if (mode == 1) {
    float s[kRefThreads];
    for (int t = 0; t < kRefThreads; ++t) {
      float v = 0.f;
      for (int g = t; g < groups; g += kRefThreads) {
        float sc = bf16_to_f32(scale[g]);
        for (int p = 0; p < kGroup / kPerWord; ++p) {
          uint32_t word = w[g * (kGroup / kPerWord) + p];
          for (int lane = 0; lane < kPerWord; ++lane) {
            float wq = bf(static_cast<float>(nibble_q(word, lane)) * sc);
            v = std::fmaf(x[g * kGroup + p * kPerWord + lane], wq, v);
          }
        }
      }
      s[t] = v;
    }
    return tree_sum(s);
  }
  double acc = 0.0;
  for (int g = 0; g < groups; ++g) {
    float sc = bf16_to_f32(scale[g]);
    for (int p = 0; p < kGroup / kPerWord; ++p) {
      uint32_t word = w[g * (kGroup / kPerWord) + p];
      for (int lane = 0; lane < kPerWord; ++lane) {
        float wq = bf(static_cast<float>(nibble_q(word, lane)) * sc);
        acc += static_cast<double>(x[g * kGroup + p * kPerWord + lane]) * static_cast<double>(wq);
      }
    }
  }
  return static_cast<float>(acc);
}

// One row of the bf16 mat-vec.  src/kimi_exec.cu:272-298.
float bf16_row(const uint16_t *w, const float *x, int cols, int mode) {
  if (mode == 1) {
    float s[kRefThreads];
    for (int t = 0; t < kRefThreads; ++t) {
      float v = 0.f;
      for (int c = t; c < cols; c += kRefThreads) v = std::fmaf(bf16_to_f32(w[c]), x[c], v);
      s[t] = v;
    }
    return tree_sum(s);
  }
  double acc = 0.0;
  for (int c = 0; c < cols; ++c) acc += static_cast<double>(bf16_to_f32(w[c])) * static_cast<double>(x[c]);
  return static_cast<float>(acc);
}

inline float silu_mul(float a, float b, int mode) {  // src/kimi_exec.cu:253-256
  if (mode == 1) return bf(bf(a / (1.0f + expf(-a))) * b);
  double s = static_cast<double>(a) / (1.0 + std::exp(-static_cast<double>(a)));
  return static_cast<float>(s * static_cast<double>(b));
}

}  // namespace

extern "C" {

int orc_num_threads() {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

void orc_set_num_threads(int n) {
#ifdef _OPENMP
  if (n > 0) omp_set_num_threads(n);
#else
  (void)n;
#endif
}

void orc_f32_to_bf16(const float *x, uint16_t *y, long n) {
  for (long i = 0; i < n; ++i) y[i] = f32_to_bf16(x[i]);
}

void orc_bf16_to_f32(const uint16_t *x, float *y, long n) {
  for (long i = 0; i < n; ++i) y[i] = bf16_to_f32(x[i]);
}

// Dequantised weight, bit-exact: bf16_rn(float(q) * float(scale)).
// src/kimi_exec.cu:311-312.  out is bf16 [rows, cols].
void orc_i4_dequant(const uint32_t *w, const uint16_t *scale, uint16_t *out, int rows, int cols) {
  const int groups = cols / kGroup, words = cols / kPerWord;
#pragma omp parallel for schedule(static)
  for (int r = 0; r < rows; ++r)
    for (int c = 0; c < cols; ++c) {
      uint32_t word = w[(size_t)r * words + c / kPerWord];
      float sc = bf16_to_f32(scale[(size_t)r * groups + c / kGroup]);
      out[(size_t)r * cols + c] = f32_to_bf16(static_cast<float>(nibble_q(word, c % kPerWord)) * sc);
    }
}

// The inverse used by the tests to build inputs: q in [-8,7] -> packed words,
// nibble = q + 8, low nibble = lowest column (compressed-tensors pack_to_int32).
void orc_i4_pack(const int8_t *q, uint32_t *w, int rows, int cols) {
  const int words = cols / kPerWord;
  for (int r = 0; r < rows; ++r)
    for (int p = 0; p < words; ++p) {
      uint32_t word = 0;
      for (int lane = 0; lane < kPerWord; ++lane)
        word |= (static_cast<uint32_t>(q[(size_t)r * cols + p * kPerWord + lane] + 8) & 0xfu) << (4 * lane);
      w[(size_t)r * words + p] = word;
    }
}

// y[r] = (round ? bf : id)(sum_c x[c] * dequant(w[r,c])).  src/kimi_exec.cu:300-323.
// round_out = 1 mirrors the reference (y is bf16-valued); 0 leaves fp32.
void orc_i4_gemv(const uint32_t *w, const uint16_t *scale, const float *x, float *y, int rows, int cols,
                 int mode, int round_out) {
  const int groups = cols / kGroup, words = cols / kPerWord;
#pragma omp parallel for schedule(static)
  for (int r = 0; r < rows; ++r) {
    float v = i4_row(w + (size_t)r * words, scale + (size_t)r * groups, x, cols, mode);
    y[r] = round_out ? bf(v) : v;
  }
}

// src/kimi_exec.cu:272-284 (round_out=1) and :286-298 (round_out=0, router logits).
void orc_bf16_gemv(const uint16_t *w, const float *x, float *y, int rows, int cols, int mode, int round_out) {
#pragma omp parallel for schedule(static)
  for (int r = 0; r < rows; ++r) {
    float v = bf16_row(w + (size_t)r * cols, x, cols, mode);
    y[r] = round_out ? bf(v) : v;
  }
}

void orc_silu_mul(const float *a, const float *b, float *y, int n, int mode) {
  for (int i = 0; i < n; ++i) y[i] = silu_mul(a[i], b[i], mode);
}

// src/kimi_exec.cu:258-270.  In place (y == x) is allowed.
void orc_rmsnorm(const float *x, const uint16_t *w, float *y, int n, float eps, int mode) {
  if (mode == 1) {
    float s[kRefThreads];
    for (int t = 0; t < kRefThreads; ++t) {
      float v = 0.f;
      for (int i = t; i < n; i += kRefThreads) v = std::fmaf(x[i], x[i], v);
      s[t] = v;
    }
    float total = tree_sum(s);
    float scale = 1.0f / sqrtf(total / n + eps);
    for (int i = 0; i < n; ++i) y[i] = bf(bf(x[i] * scale) * bf16_to_f32(w[i]));
    return;
  }
  double total = 0.0;
  for (int i = 0; i < n; ++i) total += static_cast<double>(x[i]) * x[i];
  double scale = 1.0 / std::sqrt(total / n + static_cast<double>(eps));
  for (int i = 0; i < n; ++i) y[i] = bf(static_cast<float>(x[i] * scale * bf16_to_f32(w[i])));
}

// Router for T tokens.  src/kimi_exec.cu:836-842, :377-397.
//   logit = W_r x (fp32, unrounded); s = sigmoid(logit); sel = s + bias;
//   8 rounds of argmax with strict '>' from -inf (ties -> lowest index, output in
//   descending sel order); w_k = s[id_k] / (sum + 1e-20) * routed_scale.
// margin[t] (optional) receives sel(8th) - sel(9th): tokens whose margin is below the
// caller's threshold are "ambiguous" for index parity.
void orc_router(const uint16_t *wr, const float *bias, const float *x, int T, int experts, int hidden, int topk,
                float routed_scale, uint16_t *ids, float *wts, float *margin, float *scores_out, int mode) {
#pragma omp parallel for schedule(static)
  for (int t = 0; t < T; ++t) {
    std::vector<float> s(experts), sel(experts);
    for (int e = 0; e < experts; ++e) {
      float logit = bf16_row(wr + (size_t)e * hidden, x + (size_t)t * hidden, hidden, mode);
      float sc = (mode == 1) ? 1.0f / (1.0f + expf(-logit))
                             : static_cast<float>(1.0 / (1.0 + std::exp(-static_cast<double>(logit))));
      s[e] = sc;
      sel[e] = sc + bias[e];
      if (scores_out) scores_out[(size_t)t * experts + e] = sc;
    }
    float sum = 0.f;
    std::vector<float> work(sel);
    for (int k = 0; k < topk; ++k) {
      int id = 0;
      float best = -std::numeric_limits<float>::infinity();
      for (int i = 0; i < experts; ++i)
        if (work[i] > best) best = work[i], id = i;
      ids[(size_t)t * topk + k] = static_cast<uint16_t>(id);
      wts[(size_t)t * topk + k] = s[id];
      sum += s[id];
      work[id] = -std::numeric_limits<float>::infinity();
    }
    for (int k = 0; k < topk; ++k) wts[(size_t)t * topk + k] = wts[(size_t)t * topk + k] / (sum + 1.0e-20f) * routed_scale;
    if (margin) {
      float ninth = -std::numeric_limits<float>::infinity();
      for (int i = 0; i < experts; ++i) ninth = std::max(ninth, work[i]);
      margin[t] = sel[ids[(size_t)t * topk + topk - 1]] - ninth;
    }
  }
}

// One routed expert: y = down(SiLU(gate x) * up x).  src/kimi_exec.cu:853-869.
// x, y are fp32 arrays; in ORC_REF_EXACT gate/up/mid/y are bf16-valued at each step.
// round_out: 1 = y rounded to bf16 (the reference's GEMV output), 0 = unrounded.
void orc_expert_ffn(const uint32_t *gw, const uint16_t *gs, const uint32_t *uw, const uint16_t *us,
                    const uint32_t *dw, const uint16_t *ds, const float *x, float *y, int hidden, int inter,
                    int mode, int round_out) {
  std::vector<float> g(inter), u(inter), mid(inter);
  orc_i4_gemv(gw, gs, x, g.data(), inter, hidden, mode, mode == 1);
  orc_i4_gemv(uw, us, x, u.data(), inter, hidden, mode, mode == 1);
  for (int i = 0; i < inter; ++i) mid[i] = silu_mul(g[i], u[i], mode);
  orc_i4_gemv(dw, ds, mid.data(), y, hidden, inter, mode, round_out);
}

// Dense / shared SwiGLU MLP: t = W_d (SiLU(W_g x) * W_u x).  src/kimi_exec.cu:674-686
// (the caller adds t into its running sum).  round_out as above.
void orc_bf16_mlp(const uint16_t *gw, const uint16_t *uw, const uint16_t *dw, const float *x, float *y, int hidden,
                  int ffn, int mode, int round_out) {
  std::vector<float> g(ffn), u(ffn), mid(ffn);
  orc_bf16_gemv(gw, x, g.data(), ffn, hidden, mode, mode == 1);
  orc_bf16_gemv(uw, x, u.data(), ffn, hidden, mode, mode == 1);
  for (int i = 0; i < ffn; ++i) mid[i] = silu_mul(g[i], u[i], mode);
  orc_bf16_gemv(dw, mid.data(), y, hidden, ffn, mode, round_out);
}

// One routed-MoE layer for T tokens.  src/kimi_exec.cu:836-877 applied per token.
//   out = bf( bf( sum_k w_k * y_k ) + shared )       (:868, :871, :684)
// Expert weights are given compactly: slot_of[e] is the index of expert e in the
// compact arrays (or -1 when the caller did not materialise that expert; hitting
// one returns -1).  Layout per expert: gate/up packed [inter, hidden/8], scale
// [inter, hidden/32]; down packed [hidden, inter/8], scale [hidden, inter/32].
int orc_moe_layer(const uint16_t *wr, const float *bias, const int *slot_of, const uint32_t *gw, const uint16_t *gs,
                  const uint32_t *uw, const uint16_t *us, const uint32_t *dw, const uint16_t *ds,
                  const uint16_t *sgw, const uint16_t *suw, const uint16_t *sdw, const float *x, float *out, int T,
                  int experts, int hidden, int inter, int shared_inter, int topk, float routed_scale, uint16_t *ids_out,
                  float *wts_out, int mode) {
  std::vector<uint16_t> ids((size_t)T * topk);
  std::vector<float> wts((size_t)T * topk);
  orc_router(wr, bias, x, T, experts, hidden, topk, routed_scale, ids.data(), wts.data(), nullptr, nullptr, mode);
  if (ids_out) std::memcpy(ids_out, ids.data(), ids.size() * sizeof(uint16_t));
  if (wts_out) std::memcpy(wts_out, wts.data(), wts.size() * sizeof(float));
  const size_t gu_w = (size_t)inter * hidden / kPerWord, gu_s = (size_t)inter * hidden / kGroup;
  const size_t d_w = (size_t)hidden * inter / kPerWord, d_s = (size_t)hidden * inter / kGroup;
  std::vector<float> y(hidden), sh(hidden);
  for (int t = 0; t < T; ++t) {
    const float *xt = x + (size_t)t * hidden;
    std::vector<double> acc64(hidden, 0.0);
    std::vector<float> acc32(hidden, 0.f);
    for (int k = 0; k < topk; ++k) {
      int e = ids[(size_t)t * topk + k];
      int s = slot_of[e];
      if (s < 0) return -1;
      orc_expert_ffn(gw + s * gu_w, gs + s * gu_s, uw + s * gu_w, us + s * gu_s, dw + s * d_w, ds + s * d_s, xt,
                     y.data(), hidden, inter, mode, mode == 1);
      float wk = wts[(size_t)t * topk + k];
      if (mode == 1)
        for (int i = 0; i < hidden; ++i) acc32[i] = std::fmaf(y[i], wk, acc32[i]);
      else
        for (int i = 0; i < hidden; ++i) acc64[i] += static_cast<double>(y[i]) * wk;
    }
    float *o = out + (size_t)t * hidden;
    if (sgw) {
      orc_bf16_mlp(sgw, suw, sdw, xt, sh.data(), hidden, shared_inter, mode, mode == 1);
      if (mode == 1)
        for (int i = 0; i < hidden; ++i) o[i] = bf(bf(acc32[i]) + sh[i]);
      else
        for (int i = 0; i < hidden; ++i) o[i] = bf(static_cast<float>(acc64[i] + sh[i]));
    } else {
      for (int i = 0; i < hidden; ++i) o[i] = bf(mode == 1 ? acc32[i] : static_cast<float>(acc64[i]));
    }
  }
  return 0;
}

// ---------------------------------------------------------------------------
// YaRN rotary frequencies and RoPE.  src/kimi_exec.cu:325-357.
// ---------------------------------------------------------------------------
void orc_yarn_inv_freq(float *inv_freq, int rotary, float theta, float factor, float beta_fast, float beta_slow,
                       float original_ctx) {
  const float pi = 3.14159265358979323846f;
  float dim = static_cast<float>(rotary);
  auto corr = [&](float rotations) {
    return dim * logf(original_ctx / (rotations * 2.0f * pi)) / (2.0f * logf(theta));
  };
  float low = std::max(floorf(corr(beta_fast)), 0.0f);
  float high = std::min(ceilf(corr(beta_slow)), dim - 1.0f);
  for (int pair = 0; pair < rotary / 2; ++pair) {
    float extra = powf(theta, -2.0f * static_cast<float>(pair) / dim);
    float inter = extra / factor;
    float hi = high;
    if (low == hi) hi += 0.001f;
    float ramp = std::min(1.0f, std::max(0.0f, (static_cast<float>(pair) - low) / (hi - low)));
    float mask = 1.0f - ramp;
    inv_freq[pair] = inter * (1.0f - mask) + extra * mask;
  }
}

float orc_yarn_mscale(float factor, float mscale_all_dim) {  // src/kimi_exec.cu:428
  return 0.1f * mscale_all_dim * logf(factor) + 1.0f;
}

// cos/sin table the device path consumes: c = bf(cosf(pos*f)), s = bf(sinf(pos*f)).
void orc_rope_table(const float *inv_freq, int half, int pos, float *cs) {
  for (int p = 0; p < half; ++p) {
    cs[p] = bf(cosf(pos * inv_freq[p]));
    cs[half + p] = bf(sinf(pos * inv_freq[p]));
  }
}

// Interleaved-in, de-interleaved-out rotation of one rope vector of `rotary`
// values: (in[2p], in[2p+1]) -> out[p], out[half+p].  src/kimi_exec.cu:352-356.
void orc_rope_vec(const float *in, float *out, const float *cs, int rotary) {
  int half = rotary / 2;
  for (int p = 0; p < half; ++p) {
    float c = cs[p], s = cs[half + p], x0 = in[2 * p], x1 = in[2 * p + 1];
    out[p] = bf(bf(x0 * c) - bf(x1 * s));
    out[half + p] = bf(bf(x1 * c) + bf(x0 * s));
  }
}

// ---------------------------------------------------------------------------
// MLA.  src/kimi_exec.cu:812-827 and :692-716.
// ---------------------------------------------------------------------------
struct orc_mla_dims {
  int hidden, heads, qk_nope, qk_rope, v_head, q_rank, kv_rank;
};

// Projections for one new token at `pos` (src/kimi_exec.cu:813-823).
//   q_out  [heads, qk_nope+qk_rope]  roped query (rope part de-interleaved)
//   latent [kv_rank+qk_rope]         normed c_kv then roped k_pe  (the bf16 latent-cache row)
// All outputs are bf16-valued fp32 in both modes (they are the reference's stored state).
void orc_mla_project(const orc_mla_dims *d, const uint16_t *w_qa, const uint16_t *qa_ln, const uint16_t *w_qb,
                     const uint16_t *w_kva, const uint16_t *kva_ln, const float *n, int pos, const float *inv_freq,
                     float eps, float *q_out, float *latent, int mode) {
  const int qk_head = d->qk_nope + d->qk_rope, half = d->qk_rope / 2;
  std::vector<float> qa(d->q_rank), q((size_t)d->heads * qk_head), kva(d->kv_rank + d->qk_rope), cs(d->qk_rope);
  orc_bf16_gemv(w_qa, n, qa.data(), d->q_rank, d->hidden, mode, 1);
  orc_rmsnorm(qa.data(), qa_ln, qa.data(), d->q_rank, eps, mode);
  orc_bf16_gemv(w_qb, qa.data(), q.data(), d->heads * qk_head, d->q_rank, mode, 1);
  orc_bf16_gemv(w_kva, n, kva.data(), d->kv_rank + d->qk_rope, d->hidden, mode, 1);
  orc_rmsnorm(kva.data(), kva_ln, kva.data(), d->kv_rank, eps, mode);
  orc_rope_table(inv_freq, half, pos, cs.data());
  for (int h = 0; h < d->heads; ++h) {
    std::memcpy(q_out + (size_t)h * qk_head, q.data() + (size_t)h * qk_head, d->qk_nope * sizeof(float));
    orc_rope_vec(q.data() + (size_t)h * qk_head + d->qk_nope, q_out + (size_t)h * qk_head + d->qk_nope, cs.data(),
                 d->qk_rope);
  }
  std::memcpy(latent, kva.data(), d->kv_rank * sizeof(float));
  orc_rope_vec(kva.data() + d->kv_rank, latent + d->kv_rank, cs.data(), d->qk_rope);
}

// Non-absorbed attention exactly as the reference stores and evaluates it:
// per cached token the full K [heads, qk_head] and V [heads, v_head] are
// materialised through kv_b (rounded to bf16, src/kimi_exec.cu:818-820), and the
// softmax is the three-pass form of :692-716.  latents is [seq, kv_rank+qk_rope]
// (bf16-valued fp32).  out is [heads*v_head], bf16-valued.
void orc_mla_attend_ref(const orc_mla_dims *d, const uint16_t *w_kvb, const float *q, const float *latents, int seq,
                        float softmax_mscale, float *out, int mode) {
  const int qk_head = d->qk_nope + d->qk_rope, kv_out = d->qk_nope + d->v_head;
  std::vector<float> K((size_t)seq * d->heads * qk_head), V((size_t)seq * d->heads * d->v_head);
#pragma omp parallel for schedule(static)
  for (int t = 0; t < seq; ++t) {
    const float *lat = latents + (size_t)t * (d->kv_rank + d->qk_rope);
    for (int h = 0; h < d->heads; ++h) {
      for (int i = 0; i < kv_out; ++i) {
        float v = bf(bf16_row(w_kvb + ((size_t)h * kv_out + i) * d->kv_rank, lat, d->kv_rank, mode));
        if (i < d->qk_nope) K[((size_t)t * d->heads + h) * qk_head + i] = v;
        else V[((size_t)t * d->heads + h) * d->v_head + i - d->qk_nope] = v;
      }
      for (int i = 0; i < d->qk_rope; ++i)
        K[((size_t)t * d->heads + h) * qk_head + d->qk_nope + i] = lat[d->kv_rank + i];
    }
  }
  const float inv_sqrt = 1.0f / sqrtf(static_cast<float>(qk_head));
#pragma omp parallel for schedule(static)
  for (int h = 0; h < d->heads; ++h) {
    std::vector<float> sc(seq);
    float mx = -std::numeric_limits<float>::infinity();
    for (int t = 0; t < seq; ++t) {
      const float *k = &K[((size_t)t * d->heads + h) * qk_head];
      float s;
      if (mode == 1) {
        float part[kRefThreads];
        for (int i = 0; i < kRefThreads; ++i) part[i] = i < qk_head ? q[(size_t)h * qk_head + i] * k[i] : 0.f;
        s = bf(bf(tree_sum(part)) * inv_sqrt * softmax_mscale * softmax_mscale);
      } else {
        double a = 0.0;
        for (int i = 0; i < qk_head; ++i) a += static_cast<double>(q[(size_t)h * qk_head + i]) * k[i];
        s = static_cast<float>(a * inv_sqrt * softmax_mscale * softmax_mscale);
      }
      sc[t] = s;
      mx = std::max(mx, s);
    }
    double sum = 0.0;
    float sumf = 0.f;
    if (mode == 1) {
      // :447-458 per 64-token tile: strided partials, tree, accumulated across tiles.
      for (int start = 0; start < seq; start += 64) {
        int n = std::min(64, seq - start);
        float part[kRefThreads];
        for (int i = 0; i < kRefThreads; ++i) part[i] = i < n ? expf(sc[start + i] - mx) : 0.f;
        sumf += tree_sum(part);
      }
    } else {
      for (int t = 0; t < seq; ++t) sum += std::exp(static_cast<double>(sc[t]) - mx);
    }
    for (int dd = 0; dd < d->v_head; ++dd) {
      if (mode == 1) {
        float o = 0.f;
        for (int start = 0; start < seq; start += 64) {
          int n = std::min(64, seq - start);
          float acc = 0.f;
          for (int t = start; t < start + n; ++t) {
            float p = bf(expf(sc[t] - mx) / sumf);
            acc = std::fmaf(p, V[((size_t)t * d->heads + h) * d->v_head + dd], acc);
          }
          o += acc;
        }
        out[(size_t)h * d->v_head + dd] = bf(o);
      } else {
        double o = 0.0;
        for (int t = 0; t < seq; ++t)
          o += std::exp(static_cast<double>(sc[t]) - mx) / sum * V[((size_t)t * d->heads + h) * d->v_head + dd];
        out[(size_t)h * d->v_head + dd] = bf(static_cast<float>(o));
      }
    }
  }
}

// Absorbed attention over the bf16 latent cache (the form the device path uses):
//   q_abs_h = W_UK_h^T q_nope_h,  s = (q_abs_h . c_t + q_rope_h . kpe_t) * scale,
//   o_lat_h = sum_t softmax(s)_t c_t,  out_h = W_UV_h o_lat_h.
// W_UK_h = kv_b rows [h*(nope+v), +nope), W_UV_h = rows [h*(nope+v)+nope, +v)
// (src/kimi_exec.cu:366-369).  Evaluated wide (fp64); only `out` is rounded to bf16.
// latents16 is the bf16 cache [seq, kv_rank+qk_rope].
void orc_mla_attend_absorbed(const orc_mla_dims *d, const uint16_t *w_kvb, const float *q, const uint16_t *latents16,
                             int seq, float softmax_mscale, float *out) {
  const int qk_head = d->qk_nope + d->qk_rope, kv_out = d->qk_nope + d->v_head, lat_w = d->kv_rank + d->qk_rope;
  const double scale = 1.0 / std::sqrt(static_cast<double>(qk_head)) * softmax_mscale * softmax_mscale;
#pragma omp parallel for schedule(static)
  for (int h = 0; h < d->heads; ++h) {
    std::vector<double> qabs(d->kv_rank, 0.0), sc(seq), olat(d->kv_rank, 0.0);
    for (int i = 0; i < d->qk_nope; ++i) {
      double qi = q[(size_t)h * qk_head + i];
      const uint16_t *wrow = w_kvb + ((size_t)h * kv_out + i) * d->kv_rank;
      for (int j = 0; j < d->kv_rank; ++j) qabs[j] += qi * bf16_to_f32(wrow[j]);
    }
    double mx = -std::numeric_limits<double>::infinity();
    for (int t = 0; t < seq; ++t) {
      const uint16_t *lat = latents16 + (size_t)t * lat_w;
      double a = 0.0;
      for (int j = 0; j < d->kv_rank; ++j) a += qabs[j] * bf16_to_f32(lat[j]);
      for (int i = 0; i < d->qk_rope; ++i)
        a += static_cast<double>(q[(size_t)h * qk_head + d->qk_nope + i]) * bf16_to_f32(lat[d->kv_rank + i]);
      sc[t] = a * scale;
      mx = std::max(mx, sc[t]);
    }
    double sum = 0.0;
    for (int t = 0; t < seq; ++t) {
      sc[t] = std::exp(sc[t] - mx);
      sum += sc[t];
    }
    for (int t = 0; t < seq; ++t) {
      const uint16_t *lat = latents16 + (size_t)t * lat_w;
      double p = sc[t] / sum;
      for (int j = 0; j < d->kv_rank; ++j) olat[j] += p * bf16_to_f32(lat[j]);
    }
    for (int dd = 0; dd < d->v_head; ++dd) {
      const uint16_t *wrow = w_kvb + ((size_t)h * kv_out + d->qk_nope + dd) * d->kv_rank;
      double o = 0.0;
      for (int j = 0; j < d->kv_rank; ++j) o += olat[j] * bf16_to_f32(wrow[j]);
      out[(size_t)h * d->v_head + dd] = bf(static_cast<float>(o));
    }
  }
}

// Greedy sampler: logits = bf(W_lm n); argmax with the lowest id winning ties.
// src/kimi_exec.cu:718-734, :477-493.
uint32_t orc_lm_head_argmax(const uint16_t *w, const float *n, int vocab, int hidden, int mode, float *best_out) {
  std::vector<float> logits(vocab);
  orc_bf16_gemv(w, n, logits.data(), vocab, hidden, mode, 1);
  float best = -std::numeric_limits<float>::infinity();
  uint32_t id = 0;
  for (int i = 0; i < vocab; ++i)
    if (logits[i] > best) best = logits[i], id = static_cast<uint32_t>(i);
  if (best_out) *best_out = best;
  return id;
}

// a = bf(a + b).  src/kimi_exec.cu:248-251.
void orc_add_round(float *a, const float *b, int n) {
  for (int i = 0; i < n; ++i) a[i] = bf(a[i] + b[i]);
}

}  // extern "C"
