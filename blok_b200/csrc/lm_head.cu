// Embedding row fetch and the greedy sampler: logits = bf16(W_lm n), argmax with the
// lowest id winning ties.  Reference: embed_token (src/kimi_exec.cu:651-655),
// sample_lm_head (:718-734) and argmax_k (:477-493).  The reference walks 640 tiles
// with two blocking device-to-host copies each; here the ids never leave the device.
#include "common.cuh"
#include "wgemm.h"

namespace blok {

int launch_bf16_gemv(const uint16_t *w, const uint16_t *x, uint16_t *y_bf16, float *y_f32, int rows, int cols, int T,
                     cudaStream_t stream);

// One CTA per token over bf16 logits [T, vocab].
__global__ void argmax_bf16_kernel(const uint16_t *__restrict__ logits, int vocab, uint32_t *__restrict__ ids) {
  __shared__ float sv[32];
  __shared__ int si[32];
  const uint16_t *row = logits + (size_t)blockIdx.x * vocab;
  float best = -INFINITY;
  int bi = 0x7fffffff;
  // eight logits per 16-byte load, four loads in flight per thread; a thread meets its indices in ascending order, and a
  // strict '>' keeps the lowest index (:482)
  const bool vec = vocab % 8 == 0 && (reinterpret_cast<uintptr_t>(row) & 15) == 0;
  const int units = vec ? vocab / 8 : 0;
  const uint4 *row4 = reinterpret_cast<const uint4 *>(row);
  for (int u0 = threadIdx.x; u0 < units; u0 += 4 * blockDim.x) {
    uint4 q[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const int u = u0 + k * blockDim.x;
      q[k] = u < units ? row4[u] : make_uint4(0xff80ff80u, 0xff80ff80u, 0xff80ff80u, 0xff80ff80u);  // -inf
    }
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const int i0 = (u0 + k * blockDim.x) * 8;
      const uint32_t w[4] = {q[k].x, q[k].y, q[k].z, q[k].w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float lo = bf16lo(w[j]), hi = bf16hi(w[j]);
        if (lo > best) best = lo, bi = i0 + 2 * j;
        if (hi > best) best = hi, bi = i0 + 2 * j + 1;
      }
    }
  }
  for (int i = units * 8 + threadIdx.x; i < vocab; i += blockDim.x) {
    float v = bf16_bits_to_f32(row[i]);
    if (v > best) best = v, bi = i;
  }
#pragma unroll
  for (int o = 16; o; o >>= 1) {
    float ob = __shfl_xor_sync(0xffffffffu, best, o);
    int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ob > best || (ob == best && oi < bi)) best = ob, bi = oi;
  }
  if ((threadIdx.x & 31) == 0) sv[threadIdx.x >> 5] = best, si[threadIdx.x >> 5] = bi;
  __syncthreads();
  if (threadIdx.x < 32) {
    const int nw = blockDim.x >> 5;
    best = threadIdx.x < nw ? sv[threadIdx.x] : -INFINITY;
    bi = threadIdx.x < nw ? si[threadIdx.x] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o; o >>= 1) {
      float ob = __shfl_xor_sync(0xffffffffu, best, o);
      int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ob > best || (ob == best && oi < bi)) best = ob, bi = oi;
    }
    if (threadIdx.x == 0) ids[blockIdx.x] = bi == 0x7fffffff ? 0u : (uint32_t)bi;
  }
}

// x[t, :] = table[ids[t], :]; an id outside the table raises *err (checked by the host wrapper's caller).
__global__ void embed_kernel(const uint16_t *__restrict__ table, const uint32_t *__restrict__ ids, int vocab, int hidden,
                             uint16_t *__restrict__ x, unsigned *err) {
  const uint32_t id = ids[blockIdx.x];
  if (id >= (uint32_t)vocab) {
    if (threadIdx.x == 0 && err) atomicExch(err, 1u);
    return;
  }
  const uint4 *src = reinterpret_cast<const uint4 *>(table + (size_t)id * hidden);
  uint4 *dst = reinterpret_cast<uint4 *>(x + (size_t)blockIdx.x * hidden);
  for (int i = threadIdx.x; i < hidden / 8; i += blockDim.x) dst[i] = src[i];
}

}  // namespace blok

using namespace blok;

extern "C" size_t blok_lm_head_workspace_bytes(int vocab, int T) {
  return (vocab > 0 && T > 0) ? (size_t)vocab * T * sizeof(uint16_t) : 0;
}

extern "C" int blok_lm_head_argmax(const blok_bf16_t *w, const blok_bf16_t *n, int vocab, int hidden, int T,
                                   uint32_t *ids, void *workspace, size_t workspace_bytes, blok_stream_t stream) {
  BLOK_REQUIRE(w && n && ids && workspace, BLOK_ERR_ARG, "blok_lm_head_argmax: null pointer");
  BLOK_REQUIRE(vocab > 0 && hidden > 0 && hidden % 8 == 0 && T >= 1 && T <= kWgStreamTokens, BLOK_ERR_SHAPE,
               "blok_lm_head_argmax: unsupported shape vocab=%d hidden=%d T=%d", vocab, hidden, T);
  BLOK_REQUIRE(T <= 8 || (vocab % 16 == 0 && hidden % 256 == 0), BLOK_ERR_SHAPE,
               "blok_lm_head_argmax: more than 8 rows need vocab %% 16 == 0 and hidden %% 256 == 0 (vocab=%d hidden=%d)", vocab, hidden);
  BLOK_REQUIRE(workspace_bytes >= blok_lm_head_workspace_bytes(vocab, T), BLOK_ERR_WORKSPACE,
               "blok_lm_head_argmax: workspace too small");
  uint16_t *logits = static_cast<uint16_t *>(workspace);
  // up to 8 rows: the mat-vec kernel; 9..64: one pass of the weight-streaming kernel over the table for all rows
  int rc = T <= 8 ? launch_bf16_gemv(w, n, logits, nullptr, vocab, hidden, T, (cudaStream_t)stream)
                  : launch_wgemm_rows(WG_BF16_PLAIN, w, nullptr, n, logits, nullptr, vocab, hidden, T, nullptr, 0, (cudaStream_t)stream);
  if (rc) return rc;
  argmax_bf16_kernel<<<T, 1024, 0, (cudaStream_t)stream>>>(logits, vocab, ids);
  return launch_status("argmax_bf16_kernel");
}

extern "C" int blok_embed(const blok_bf16_t *table, const uint32_t *ids, int vocab, int hidden, int T, blok_bf16_t *x,
                          blok_stream_t stream) {
  BLOK_REQUIRE(table && ids && x, BLOK_ERR_ARG, "blok_embed: null pointer");
  BLOK_REQUIRE(vocab > 0 && hidden > 0 && hidden % 8 == 0 && T >= 0, BLOK_ERR_SHAPE, "blok_embed: unsupported shape");
  if (T == 0) return BLOK_OK;
  embed_kernel<<<T, 256, 0, (cudaStream_t)stream>>>(table, ids, vocab, hidden, x, nullptr);
  return launch_status("embed_kernel");
}
