// Pinning harness: compiles the reference executor's single translation unit
// from where it lies (found through -I <reference>/src at build time; the source
// is never copied into this repository) and exposes extern "C" launchers for
// its kernels, so that the CPU oracle can be checked against the reference's
// own arithmetic on a GPU.  Test infrastructure only.
//
// The reference does not compile as shipped with CUDA 12.9: it uses
// CUDART_INF_F / CUDART_PI_F without including <math_constants.h>, and uses
// CUDART_INF_F in host code.  oracle/build.py passes the two macros on the
// command line; nothing in the reference source is edited.
#define main blok_ref_main
#include "kimi_exec.cu"
#undef main

namespace {
int done() {
  cudaError_t e = cudaDeviceSynchronize();
  return e == cudaSuccess ? 0 : -(int)e;
}
}  // namespace

extern "C" {

// src/kimi_exec.cu:300-323 launched as at :689 (one block per row, 256 threads).
int ref_matvec_i4(const std::uint32_t *w, const __nv_bfloat16 *scale, const float *x, float *y, int rows, int cols) {
  for (int r = 0; r < rows; r += EXPERT_TILE) {
    int n = std::min(EXPERT_TILE, rows - r);
    matvec_i4_bf16_scale_k<<<n, 256>>>(w + (size_t)r * (cols / I4_PER_WORD), scale + (size_t)r * (cols / I4_GROUP), x,
                                       y + r, n, cols);
  }
  return done();
}

// :272-284 as at :659.
int ref_matvec_bf16(const __nv_bfloat16 *w, const float *x, float *y, int rows, int cols) {
  for (int r = 0; r < rows; r += EXPERT_TILE) {
    int n = std::min(EXPERT_TILE, rows - r);
    matvec_bf16_k<<<n, 256>>>(w + (size_t)r * cols, x, y + r, n, cols);
  }
  return done();
}

// :286-298 as at :666 (unrounded fp32 output).
int ref_matvec_bf16_f32(const __nv_bfloat16 *w, const float *x, float *y, int rows, int cols) {
  for (int r = 0; r < rows; r += EXPERT_TILE) {
    int n = std::min(EXPERT_TILE, rows - r);
    matvec_bf16_f32_k<<<n, 256>>>(w + (size_t)r * cols, x, y + r, cols);
  }
  return done();
}

int ref_silu_mul(const float *a, const float *b, float *y, int n) {  // :253 as at :861
  silu_mul_k<<<(n + 255) / 256, 256>>>(a, b, y, n);
  return done();
}

int ref_rmsnorm(const float *x, const __nv_bfloat16 *w, float *y, int n) {  // :258 as at :812
  rmsnorm_k<<<1, 256>>>(x, w, y, n);
  return done();
}

int ref_add(float *a, const float *b, int n) {  // :248 as at :827
  add_k<<<(n + 255) / 256, 256>>>(a, b, n);
  return done();
}

// Router tail as at :839-842.  logits [384] fp32 is overwritten with the sigmoid
// scores; select [384] is scratch; bias is bf16 [384].
int ref_router_tail(float *logits, float *select, const __nv_bfloat16 *bias, std::uint16_t *expert, float *weight) {
  sigmoid_k<<<(EXPERTS + 255) / 256, 256>>>(logits, EXPERTS);
  if (cudaMemcpy(select, logits, EXPERTS * sizeof(float), cudaMemcpyDeviceToDevice) != cudaSuccess) return -1;
  add_bf16_k<<<(EXPERTS + 255) / 256, 256>>>(select, bias, EXPERTS);
  router_topk_k<<<1, EXPERTS>>>(logits, select, expert, weight);
  return done();
}

int ref_expert_accum(const float *y, const float *w, int slot, float *out, int n) {  // :399 as at :868
  expert_accum_k<<<(n + 255) / 256, 256>>>(y, w, slot, out, n);
  return done();
}

int ref_round_bf16(float *x, int n) {  // :404 as at :871
  round_bf16_k<<<(n + 255) / 256, 256>>>(x, n);
  return done();
}

// :346-357 as at :821-823: q, k are [64*192]; qr, kr must hold copies of q, k.
int ref_rope(const float *q, const float *k, float *qr, float *kr, int pos) {
  if (cudaMemcpy(qr, q, K_DIM * sizeof(float), cudaMemcpyDeviceToDevice) != cudaSuccess) return -1;
  if (cudaMemcpy(kr, k, K_DIM * sizeof(float), cudaMemcpyDeviceToDevice) != cudaSuccess) return -1;
  rope_k<<<(HEADS * QK_ROPE / 2 + 255) / 256, 256>>>(q, k, qr, kr, pos, HEADS, QK_HEAD, QK_ROPE);
  return done();
}

int ref_split_kv(const float *kv, float *k, float *v, const float *kpe) {  // :819-820
  split_kv_k<<<(HEADS * (QK_NOPE + V_HEAD) + 255) / 256, 256>>>(kv, k, v);
  k_rope_fill_k<<<(HEADS * QK_ROPE + 255) / 256, 256>>>(k, kpe);
  return done();
}

// The launch sequence of tiled_attention (:692-716) with the K and V histories
// resident in device memory (K [seq, 64*192], V [seq, 64*128], fp32) instead of
// being re-read tile by tile from storage.  score [64*tile], hmax [64], hsum [64]
// are scratch.
int ref_tiled_attention(const float *K, const float *V, int seq, int tile, const float *q, float *out, float *score,
                        float *hmax, float *hsum) {
  fill_k<<<1, 256>>>(hmax, -__builtin_huge_valf(), HEADS);
  if (cudaMemset(out, 0, V_DIM * sizeof(float)) != cudaSuccess) return -1;
  for (int start = 0; start < seq; start += tile) {
    int n = std::min(tile, seq - start);
    attn_tile_score_k<<<dim3(HEADS, n), 256>>>(q, K + (size_t)start * K_DIM, score, n);
    attn_tile_max_k<<<HEADS, 256>>>(score, hmax, n);
  }
  if (cudaMemset(hsum, 0, HEADS * sizeof(float)) != cudaSuccess) return -1;
  for (int start = 0; start < seq; start += tile) {
    int n = std::min(tile, seq - start);
    attn_tile_score_k<<<dim3(HEADS, n), 256>>>(q, K + (size_t)start * K_DIM, score, n);
    attn_tile_sum_k<<<HEADS, 256>>>(score, hmax, hsum, n);
  }
  for (int start = 0; start < seq; start += tile) {
    int n = std::min(tile, seq - start);
    attn_tile_score_k<<<dim3(HEADS, n), 256>>>(q, K + (size_t)start * K_DIM, score, n);
    attn_tile_accum_k<<<dim3(HEADS, (V_HEAD + 255) / 256), 256>>>(score, V + (size_t)start * V_DIM, hmax, hsum, out, n);
  }
  attn_finish_k<<<(V_DIM + 255) / 256, 256>>>(out);
  return done();
}

int ref_argmax(const float *x, std::uint32_t *id, int n) {  // :477 as at :726
  argmax_k<<<1, 256>>>(x, id, n);
  return done();
}

}  // extern "C"
