// Routed-MoE layer handle and the batch-1 decode path.
// Reference: the MoE branch of the layer body, src/kimi_exec.cu:836-875.
#include <algorithm>
#include <cstdlib>
#include <new>
#include <string>

#include "common.cuh"
#include "moe_layer.h"
#include "wgemm.h"

namespace blok {

int launch_bf16_gemv(const uint16_t *w, const uint16_t *x, uint16_t *y_bf16, float *y_f32, int rows, int cols, int T,
                     cudaStream_t stream);
int launch_bf16_gateup(const uint16_t *gate, const uint16_t *up, const uint16_t *x, uint16_t *mid, int ffn, int cols,
                       int T, cudaStream_t stream);
int launch_router_topk(const float *logits, const float *bias, int T, int experts, int topk, float routed_scale,
                       uint16_t *ids, float *wts, int *local_ids, int expert_base, cudaStream_t stream);
int launch_i4_gateup(const uint32_t *gate_w, const uint16_t *gate_s, const uint32_t *up_w, const uint16_t *up_s,
                     const uint16_t *x, const int *slot_expert, uint16_t *mid, int hidden, int inter, int slots,
                     cudaStream_t stream);
int launch_i4_down(const uint32_t *down_w, const uint16_t *down_s, const uint16_t *mid, const int *slot_expert,
                   const float *wts, const uint16_t *addend, uint16_t *out, int hidden, int inter, int slots,
                   cudaStream_t stream);

int fused_plan(const blok_moe_weights &w, FusedPlan *plan);
int batched_alloc(blok_moe_layer *L);
int launch_moe_decode_fused(blok_moe_layer *L, const uint16_t *x, uint16_t *y, uint16_t *ids_out, float *wts_out,
                            cudaStream_t stream, unsigned *err_host = nullptr, float *part_out = nullptr,
                            uint16_t *shared_out = nullptr);

static size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

}  // namespace blok

using namespace blok;

extern "C" int blok_moe_layer_create(const blok_moe_weights *w, int max_tokens, blok_moe_layer_t **out) {
  BLOK_REQUIRE(w && out, BLOK_ERR_ARG, "blok_moe_layer_create: null pointer");
  BLOK_REQUIRE(max_tokens >= 1, BLOK_ERR_ARG, "blok_moe_layer_create: max_tokens must be >= 1");
  BLOK_REQUIRE(w->hidden > 0 && w->hidden % 256 == 0 && w->inter > 0 && w->inter % 256 == 0 && w->hidden <= 32768 &&
                   w->inter <= 32768,
               BLOK_ERR_SHAPE, "blok_moe_layer_create: hidden %d / inter %d must be multiples of 256 (<= 32768)",
               w->hidden, w->inter);
  BLOK_REQUIRE(w->experts > 0 && w->experts <= 1024 && w->topk >= 1 && w->topk <= 16 && w->topk <= w->experts,
               BLOK_ERR_SHAPE, "blok_moe_layer_create: experts %d / topk %d unsupported", w->experts, w->topk);
  BLOK_REQUIRE(w->experts_local >= 0 && w->expert_base >= 0 && w->expert_base + w->experts_local <= w->experts,
               BLOK_ERR_SHAPE, "blok_moe_layer_create: local expert range [%d, %d) outside [0, %d)", w->expert_base,
               w->expert_base + w->experts_local, w->experts);
  BLOK_REQUIRE(w->shared_inter >= 0 && w->shared_inter % 32 == 0, BLOK_ERR_SHAPE,
               "blok_moe_layer_create: shared_inter %d must be a multiple of 32", w->shared_inter);
  BLOK_REQUIRE(w->router_w && w->router_bias, BLOK_ERR_ARG, "blok_moe_layer_create: router weights missing");
  if (w->experts_local > 0)
    BLOK_REQUIRE(w->gate_w && w->gate_s && w->up_w && w->up_s && w->down_w && w->down_s, BLOK_ERR_ARG,
                 "blok_moe_layer_create: routed expert weights missing");
  if (w->shared_inter > 0)
    BLOK_REQUIRE(w->shared_gate && w->shared_up && w->shared_down, BLOK_ERR_ARG,
                 "blok_moe_layer_create: shared expert weights missing");
  blok_moe_layer *L = new (std::nothrow) blok_moe_layer();
  BLOK_REQUIRE(L, BLOK_ERR_ARG, "blok_moe_layer_create: out of host memory");
  L->w = *w;
  L->max_tokens = max_tokens;
  {
    int rc = fused_plan(*w, &L->plan);
    if (rc) {
      delete L;
      return rc;
    }
    const char *impl = std::getenv("BLOK_MOE_DECODE_IMPL");  // "multi" forces the multi-kernel path (for comparison)
    L->use_fused = L->plan.enabled && !(impl && std::string(impl) == "multi");
  }
  // decode workspace carve-up
  size_t off = 0;
  auto take = [&](size_t bytes) {
    size_t at = off;
    off = align_up(off + bytes, 256);
    return at;
  };
  size_t o_logits = take((size_t)max_tokens * w->experts * sizeof(float));
  size_t o_ids = take((size_t)max_tokens * w->topk * sizeof(uint16_t));
  size_t o_local = take((size_t)max_tokens * w->topk * sizeof(int));
  size_t o_wts = take((size_t)max_tokens * w->topk * sizeof(float));
  size_t o_mid = take((size_t)w->topk * w->inter * sizeof(uint16_t));
  size_t o_smid = take((size_t)(w->shared_inter ? w->shared_inter : 1) * 8 * sizeof(uint16_t));
  size_t o_sout = take((size_t)w->hidden * 8 * sizeof(uint16_t));
  size_t o_iox = take((size_t)w->hidden * sizeof(uint16_t));
  size_t o_ioy = take((size_t)w->hidden * sizeof(uint16_t));
  const blok::FusedPlan &pl = L->plan;
  size_t o_flog = 0, o_fmid = 0, o_fys = 0, o_pR = 0, o_route = 0, o_pA = 0, o_pB = 0, o_pC2 = 0, o_cnt = 0, n_cnt = 0;
  if (pl.enabled) {
    L->f_mid_stride = (int)align_up((size_t)std::max(w->inter, w->shared_inter), 64);
    o_fmid = take((size_t)(w->topk + 1) * L->f_mid_stride * 4);
    o_flog = take((size_t)w->experts * 16);  // two tagged values per expert
    o_fys = take((size_t)(w->topk + 1) * w->hidden * 2 * sizeof(float));
    o_route = take(32 * sizeof(float));
    o_pR = take((size_t)pl.nrbR * pl.cprR * 16 * 2 * sizeof(float));
    o_pA = take((size_t)std::max(pl.nrbA, 1) * pl.cprA * 16 * 2 * sizeof(float));
    o_pB = take((size_t)pl.nrbB * pl.cprB * 16 * 2 * sizeof(float));
    o_pC2 = take((size_t)std::max(pl.nrbC2, 1) * pl.cprC2 * 16 * 2 * sizeof(float));
    n_cnt = (size_t)pl.nrbR + pl.nrbA + pl.nrbB + pl.nrbC2 + w->hidden / 16 + 8 + 64;  // + 64: the last block holds at least 64 words
    o_cnt = take(n_cnt * sizeof(unsigned));
  }
  const char *trace_env = std::getenv("BLOK_MOE_TRACE");
  const bool want_trace = pl.enabled && trace_env && trace_env[0] == '1';
  size_t o_trace = want_trace ? take(((size_t)pl.grid + 1) * 48 * sizeof(long long)) : 0;  // 16 stamps per CTA, then 2 per warp
  L->ws_bytes = off;
  cudaError_t e = cudaMalloc(&L->ws, L->ws_bytes);
  if (e != cudaSuccess) {
    delete L;
    return cuda_fail(e, "cudaMalloc(moe layer workspace)");
  }
  e = cudaMemset(L->ws, 0, L->ws_bytes);
  if (e != cudaSuccess) {
    cudaFree(L->ws);
    delete L;
    return cuda_fail(e, "cudaMemset(moe layer workspace)");
  }
  unsigned char *b = static_cast<unsigned char *>(L->ws);
  L->logits = reinterpret_cast<float *>(b + o_logits);
  L->ids = reinterpret_cast<uint16_t *>(b + o_ids);
  L->local_ids = reinterpret_cast<int *>(b + o_local);
  L->wts = reinterpret_cast<float *>(b + o_wts);
  L->mid = reinterpret_cast<uint16_t *>(b + o_mid);
  L->shared_mid = reinterpret_cast<uint16_t *>(b + o_smid);
  L->shared_out = reinterpret_cast<uint16_t *>(b + o_sout);
  L->io_x = reinterpret_cast<uint16_t *>(b + o_iox);
  L->io_y = reinterpret_cast<uint16_t *>(b + o_ioy);
  if (cudaMallocHost(&L->io_err_host, sizeof(unsigned)) != cudaSuccess) {
    cudaGetLastError();
    L->io_err_host = nullptr;  // the host-buffer entry point then checks with a separate copy
  } else {
    *L->io_err_host = 0;
  }
  if (pl.enabled) {
    L->f_mid = reinterpret_cast<uint16_t *>(b + o_fmid);
    L->f_logits_t = reinterpret_cast<float *>(b + o_flog);
    L->f_ys = reinterpret_cast<float *>(b + o_fys);
    L->f_route_ids = reinterpret_cast<int *>(b + o_route);
    L->f_route_wts = reinterpret_cast<float *>(b + o_route) + 16;
    L->f_partR = reinterpret_cast<float *>(b + o_pR);
    L->f_partA = reinterpret_cast<float *>(b + o_pA);
    L->f_partB = reinterpret_cast<float *>(b + o_pB);
    L->f_partC2 = reinterpret_cast<float *>(b + o_pC2);
    unsigned *c = reinterpret_cast<unsigned *>(b + o_cnt);
    L->f_counters = c;
    L->f_counters_bytes = n_cnt * sizeof(unsigned);
    L->f_ctrl = c;
    c += 8;
    L->f_cntR = c; c += pl.nrbR;
    L->f_cntA = c; c += pl.nrbA;
    L->f_cntB = c; c += pl.nrbB;
    L->f_cntC2 = c; c += pl.nrbC2;
    L->f_cntOut = c;
    if (want_trace) L->f_trace = reinterpret_cast<long long *>(b + o_trace);
  }
  if (max_tokens > 1) {
    int rc = batched_alloc(L);
    if (rc) {
      cudaFree(L->ws);
      delete L;
      return rc;
    }
  }
  *out = L;
  return BLOK_OK;
}

extern "C" int blok_moe_layer_destroy(blok_moe_layer_t *L) {
  if (!L) return BLOK_OK;
  cudaError_t e = L->ws ? cudaFree(L->ws) : cudaSuccess;
  if (L->io_err_host) cudaFreeHost(L->io_err_host);
  if (L->bws) {
    cudaError_t e2 = cudaFree(L->bws);
    if (e == cudaSuccess) e = e2;
  }
  delete L;
  return e == cudaSuccess ? BLOK_OK : cuda_fail(e, "cudaFree(moe layer workspace)");
}

extern "C" int blok_moe_decode(blok_moe_layer_t *L, const blok_bf16_t *x, blok_bf16_t *y, uint16_t *ids_out,
                               float *wts_out, blok_stream_t stream_) {
  BLOK_REQUIRE(L && x && y, BLOK_ERR_ARG, "blok_moe_decode: null pointer");
  const blok_moe_weights &w = L->w;
  BLOK_REQUIRE(w.experts_local == w.experts && w.expert_base == 0, BLOK_ERR_ROUTE,
               "blok_moe_decode: needs every expert local (have [%d, %d) of %d)", w.expert_base,
               w.expert_base + w.experts_local, w.experts);
  cudaStream_t stream = (cudaStream_t)stream_;
  if (L->use_fused) return launch_moe_decode_fused(L, x, y, ids_out, wts_out, stream);
  int rc = launch_bf16_gemv(w.router_w, x, nullptr, L->logits, w.experts, w.hidden, 1, stream);
  if (rc) return rc;
  rc = launch_router_topk(L->logits, w.router_bias, 1, w.experts, w.topk, w.routed_scale, L->ids, L->wts, L->local_ids,
                          w.expert_base, stream);
  if (rc) return rc;
  const uint16_t *addend = nullptr;
  if (w.shared_inter > 0) {
    rc = launch_bf16_gateup(w.shared_gate, w.shared_up, x, L->shared_mid, w.shared_inter, w.hidden, 1, stream);
    if (rc) return rc;
    rc = launch_bf16_gemv(w.shared_down, L->shared_mid, L->shared_out, nullptr, w.hidden, w.shared_inter, 1, stream);
    if (rc) return rc;
    addend = L->shared_out;
  }
  rc = launch_i4_gateup(w.gate_w, w.gate_s, w.up_w, w.up_s, x, L->local_ids, L->mid, w.hidden, w.inter, w.topk, stream);
  if (rc) return rc;
  rc = launch_i4_down(w.down_w, w.down_s, L->mid, L->local_ids, L->wts, addend, y, w.hidden, w.inter, w.topk, stream);
  if (rc) return rc;
  if (ids_out)
    BLOK_CUDA(cudaMemcpyAsync(ids_out, L->ids, w.topk * sizeof(uint16_t), cudaMemcpyDeviceToDevice, stream));
  if (wts_out) BLOK_CUDA(cudaMemcpyAsync(wts_out, L->wts, w.topk * sizeof(float), cudaMemcpyDeviceToDevice, stream));
  return BLOK_OK;
}

extern "C" int blok_moe_decode_partial(blok_moe_layer_t *L, const blok_bf16_t *x, float *part, blok_bf16_t *shared_out,
                                       uint16_t *ids_out, float *wts_out, blok_stream_t stream_) {
  BLOK_REQUIRE(L && x && part && shared_out, BLOK_ERR_ARG, "blok_moe_decode_partial: null pointer");
  BLOK_REQUIRE(L->use_fused && L->w.shared_inter > 0, BLOK_ERR_STATE,
               "blok_moe_decode_partial: this layer has no fused decode kernel (blok_moe_layer_has_partial)");
  return launch_moe_decode_fused(L, x, nullptr, ids_out, wts_out, (cudaStream_t)stream_, nullptr, part, shared_out);
}

extern "C" int blok_moe_layer_has_partial(blok_moe_layer_t *L) { return L && L->use_fused && L->w.shared_inter > 0 ? 1 : 0; }

extern "C" int blok_moe_layer_check(blok_moe_layer_t *L, blok_stream_t stream_) {
  BLOK_REQUIRE(L, BLOK_ERR_ARG, "blok_moe_layer_check: null pointer");
  cudaStream_t stream = (cudaStream_t)stream_;
  BLOK_CUDA(cudaStreamSynchronize(stream));
  unsigned tc_err = 0;
  if (int rc = wgemm_tc_take_error(&tc_err)) return rc;
  if (tc_err) {
    set_error("blok_moe_batched: a tensor-core GEMM tile gave up waiting for its MMAs");
    return BLOK_ERR_TIMEOUT;
  }
  if (!L->f_ctrl) return BLOK_OK;
  unsigned err = 0;
  BLOK_CUDA(cudaMemcpy(&err, L->f_ctrl + 5, sizeof(err), cudaMemcpyDeviceToHost));
  if (err == 0) return BLOK_OK;
  // a bounded wait inside the fused kernel gave up: clear every counter so that the handle stays usable
  BLOK_CUDA(cudaMemset(L->ws, 0, L->ws_bytes));  // counters, launch tags and the epoch all restart together
  set_error("blok_moe_decode: device-side wait %u timed out (1 = routing, 2 = mid values)", err);
  return BLOK_ERR_TIMEOUT;
}

extern "C" int blok_moe_layer_debug_set_error(blok_moe_layer_t *L, unsigned code, blok_stream_t stream) {
  BLOK_REQUIRE(L, BLOK_ERR_ARG, "blok_moe_layer_debug_set_error: null pointer");
  BLOK_REQUIRE(L->f_ctrl, BLOK_ERR_STATE, "blok_moe_layer_debug_set_error: this layer has no fused decode kernel (no error word)");
  BLOK_CUDA(cudaMemcpyAsync(L->f_ctrl + 5, &code, sizeof(code), cudaMemcpyHostToDevice, (cudaStream_t)stream));
  BLOK_CUDA(cudaStreamSynchronize((cudaStream_t)stream));
  return BLOK_OK;
}

// The device address of a host buffer the GPU can write directly (pinned memory), or NULL.  The last answer is kept:
// a caller that reuses its buffers pays for the query once.
static void *mapped_address(blok_moe_layer *L, const void *host) {
  if (host == L->io_last_host) return L->io_last_dev;
  cudaPointerAttributes at;
  void *dev = nullptr;
  if (cudaPointerGetAttributes(&at, host) == cudaSuccess && at.type == cudaMemoryTypeHost) dev = at.devicePointer;
  else cudaGetLastError();
  L->io_last_host = host;
  L->io_last_dev = dev;
  return dev;
}

extern "C" int blok_moe_decode_host(blok_moe_layer_t *L, const blok_bf16_t *x_host, blok_bf16_t *y_host,
                                    blok_stream_t stream_) {
  BLOK_REQUIRE(L && x_host && y_host, BLOK_ERR_ARG, "blok_moe_decode_host: null pointer");
  cudaStream_t stream = (cudaStream_t)stream_;
  const size_t bytes = (size_t)L->w.hidden * sizeof(uint16_t);
  BLOK_CUDA(cudaMemcpyAsync(L->io_x, x_host, bytes, cudaMemcpyHostToDevice, stream));
  const blok_moe_weights &w = L->w;
  if (L->use_fused && L->io_err_host && w.experts_local == w.experts && w.expert_base == 0) {
    // One copy in, one launch, one synchronisation: when y_host is pinned the kernel's finishers store the result
    // straight into it (14 KB over the bus while the kernel still runs), and the last CTA to leave stores the launch's
    // error word into a pinned word of the handle; the host reads both after the stream has drained.
    uint16_t *y_dev = static_cast<uint16_t *>(mapped_address(L, y_host));
    void *err_dev = nullptr;
    if (cudaHostGetDevicePointer(&err_dev, L->io_err_host, 0) != cudaSuccess) {
      cudaGetLastError();
      err_dev = nullptr;
    }
    if (err_dev) {
      *L->io_err_host = 0;
      int rc = launch_moe_decode_fused(L, L->io_x, y_dev ? y_dev : L->io_y, nullptr, nullptr, stream, static_cast<unsigned *>(err_dev));
      if (rc) return rc;
      if (!y_dev) BLOK_CUDA(cudaMemcpyAsync(y_host, L->io_y, bytes, cudaMemcpyDeviceToHost, stream));  // pageable: staged copy
      BLOK_CUDA(cudaStreamSynchronize(stream));
      if (*L->io_err_host == 0) return BLOK_OK;
      return blok_moe_layer_check(L, stream_);  // a wait gave up: report it and reset the handle
    }
  }
  int rc = blok_moe_decode(L, L->io_x, L->io_y, nullptr, nullptr, stream_);
  if (rc) return rc;
  BLOK_CUDA(cudaMemcpyAsync(y_host, L->io_y, bytes, cudaMemcpyDeviceToHost, stream));
  return blok_moe_layer_check(L, stream_);
}

extern "C" int blok_moe_layer_trace(blok_moe_layer_t *L, long long *host_out, int max_entries) {
  BLOK_REQUIRE(L && host_out, BLOK_ERR_ARG, "blok_moe_layer_trace: null pointer");
  if (!L->f_trace) return 0;
  int n = (L->plan.grid + 1) * 48;
  if (n > max_entries) n = max_entries;
  BLOK_CUDA(cudaDeviceSynchronize());
  BLOK_CUDA(cudaMemcpy(host_out, L->f_trace, (size_t)n * sizeof(long long), cudaMemcpyDeviceToHost));
  return n;
}
