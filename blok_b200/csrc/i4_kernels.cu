// INT4 (W4A16) kernels: dequant probe, mat-vec, and the single-expert SwiGLU FFN.
// Reference arithmetic: src/kimi_exec.cu:300-323 (matvec_i4_bf16_scale_k),
// :253-256 (silu_mul_k), :853-869 (per-slot body of the routed-expert loop).
#include <mutex>

#include <cstdlib>
#include <cstring>

#include "i4_mma.cuh"

namespace blok {

// ---------------------------------------------------------------------------
// Dequant probe: one thread per packed word, 8 bf16 out (one 16-byte store).
// ---------------------------------------------------------------------------
__global__ void i4_dequant_kernel(const uint32_t *__restrict__ w, const uint16_t *__restrict__ scale,
                                  uint4 *__restrict__ out, long words, int words_per_row) {
  long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= words) return;
  long r = i / words_per_row;
  int p = (int)(i - r * words_per_row);
  uint32_t word = w[i];
  float sc = bf16_bits_to_f32(scale[r * (words_per_row / 4) + p / 4]);
  uint32_t o[4];
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    float q0 = (float)((int)((word >> (8 * k)) & 0xf) - 8);
    float q1 = (float)((int)((word >> (8 * k + 4)) & 0xf) - 8);
    o[k] = pack_bf16x2(q0 * sc, q1 * sc);
  }
  out[i] = make_uint4(o[0], o[1], o[2], o[3]);
}

// ---------------------------------------------------------------------------
// Scalar mat-vec for arbitrary rows and cols % 32 == 0: one warp per row, the
// reference's per-weight rounding bf16(q * scale) kept.
// ---------------------------------------------------------------------------
template <typename XT>
__device__ __forceinline__ float load_x(const XT *x, int c);
template <>
__device__ __forceinline__ float load_x<float>(const float *x, int c) {
  return x[c];
}
template <>
__device__ __forceinline__ float load_x<uint16_t>(const uint16_t *x, int c) {
  return bf16_bits_to_f32(x[c]);
}

template <typename XT, typename YT>
__global__ void i4_gemv_scalar_kernel(const uint32_t *__restrict__ w, const uint16_t *__restrict__ scale,
                                      const XT *__restrict__ x, YT *__restrict__ y, int rows, int cols) {
  int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (warp >= rows) return;
  const int groups = cols / 32;
  const uint4 *wr = reinterpret_cast<const uint4 *>(w + (size_t)warp * (cols / 8));
  const uint16_t *sr = scale + (size_t)warp * groups;
  float acc = 0.f;
  for (int g = lane; g < groups; g += 32) {
    uint4 v = ldg_stream(wr + g);
    float sc = bf16_bits_to_f32(sr[g]);
    const uint32_t words[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int p = 0; p < 4; ++p)
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        float q = (float)((int)((words[p] >> (4 * k)) & 0xf) - 8);
        acc = fmaf(load_x<XT>(x, g * 32 + p * 8 + k), round_bf16(q * sc), acc);
      }
  }
  acc = warp_sum(acc);
  if (lane == 0) {
    if constexpr (sizeof(YT) == 2) y[warp] = f32_to_bf16_bits(acc);
    else y[warp] = round_bf16(acc);
  }
}

// ---------------------------------------------------------------------------
// Tensor-core mat-vec: CTA = 16 rows, warps split K.
// ---------------------------------------------------------------------------
constexpr int kMaxWarps = 16;

template <int BATCH, typename YT>
__global__ void __launch_bounds__(kMaxWarps * 32)
    i4_gemv16_kernel(const uint32_t *__restrict__ w, const uint16_t *__restrict__ scale,
                     const uint16_t *__restrict__ x, YT *__restrict__ y, int cols, int nbatch) {
  extern __shared__ __align__(16) unsigned char smem[];
  __shared__ float partial[kMaxWarps][16];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarps = blockDim.x >> 5;
  const int g = lane >> 2, t = lane & 3;
  I4Stage st = i4_stage_carve(smem, cols, BATCH);
  stage_x_i4(reinterpret_cast<const uint4 *>(x), st, cols, BATCH, tid, blockDim.x);
  __syncthreads();
  const int row0 = blockIdx.x * 16;
  const size_t wrow = cols / 32;  // uint4 per row == scale entries per row
  const uint4 *w_lo = reinterpret_cast<const uint4 *>(w) + (size_t)(row0 + g) * wrow;
  const uint4 *w_hi = w_lo + 8 * wrow;
  const uint16_t *s_sel = scale + (size_t)(row0 + g + 8 * (t >> 1)) * wrow + 2 * (t & 1);
  XFragLane xl = xfrag_lane(st, lane, BATCH);
  float acc = i4_rows16_accumulate<BATCH>(w_lo, w_hi, s_sel, xl, st.xsum, warp * nbatch * BATCH, nbatch, lane);
  acc += __shfl_xor_sync(0xffffffffu, acc, 1);
  if ((t & 1) == 0) partial[warp][g + 8 * (t >> 1)] = acc;
  __syncthreads();
  if (tid < 16) {
    float v = 0.f;
    for (int wi = 0; wi < nwarps; ++wi) v += partial[wi][tid];
    if constexpr (sizeof(YT) == 2) y[row0 + tid] = f32_to_bf16_bits(v);
    else y[row0 + tid] = round_bf16(v);
  }
}

// ---------------------------------------------------------------------------
// gate/up with fused SiLU*up.  grid = (inter/8, slots).  A-low rows are 8 gate
// rows, A-high rows the same 8 up rows, so the SiLU*up epilogue needs no second
// pass.  slot_expert (device, may be NULL = identity) maps slot -> local expert.
// mid is bf16 [slots, inter] in natural order.
// ---------------------------------------------------------------------------
template <int BATCH>
__global__ void __launch_bounds__(kMaxWarps * 32)
    i4_gateup_kernel(const uint32_t *__restrict__ gate_w, const uint16_t *__restrict__ gate_s,
                     const uint32_t *__restrict__ up_w, const uint16_t *__restrict__ up_s,
                     const uint16_t *__restrict__ x, const int *__restrict__ slot_expert, uint16_t *__restrict__ mid,
                     int cols, int inter, int nbatch) {
  extern __shared__ __align__(16) unsigned char smem[];
  __shared__ float partial[kMaxWarps][16];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarps = blockDim.x >> 5;
  const int g = lane >> 2, t = lane & 3;
  I4Stage st = i4_stage_carve(smem, cols, BATCH);
  stage_x_i4(reinterpret_cast<const uint4 *>(x), st, cols, BATCH, tid, blockDim.x);
  __syncthreads();
  const int slot = blockIdx.y;
  const int e = slot_expert ? slot_expert[slot] : slot;
  const int row0 = blockIdx.x * 8;
  const size_t wrow = cols / 32;
  const size_t ebase = (size_t)e * inter * wrow;
  const uint4 *w_lo = reinterpret_cast<const uint4 *>(gate_w) + ebase + (size_t)(row0 + g) * wrow;
  const uint4 *w_hi = reinterpret_cast<const uint4 *>(up_w) + ebase + (size_t)(row0 + g) * wrow;
  const uint16_t *s_sel = ((t >> 1) ? up_s : gate_s) + ebase + (size_t)(row0 + g) * wrow + 2 * (t & 1);
  XFragLane xl = xfrag_lane(st, lane, BATCH);
  float acc = i4_rows16_accumulate<BATCH>(w_lo, w_hi, s_sel, xl, st.xsum, warp * nbatch * BATCH, nbatch, lane);
  acc += __shfl_xor_sync(0xffffffffu, acc, 1);
  if ((t & 1) == 0) partial[warp][g + 8 * (t >> 1)] = acc;
  __syncthreads();
  if (tid < 8) {
    float gv = 0.f, uv = 0.f;
    for (int wi = 0; wi < nwarps; ++wi) {
      gv += partial[wi][tid];
      uv += partial[wi][8 + tid];
    }
    // the reference rounds each GEMV output (:322) and both SiLU steps (:255)
    gv = round_bf16(gv);
    uv = round_bf16(uv);
    float m = round_bf16(round_bf16(gv / (1.0f + expf(-gv))) * uv);
    mid[(size_t)slot * inter + row0 + tid] = f32_to_bf16_bits(m);
  }
}

// ---------------------------------------------------------------------------
// down projection + weighted combine.  grid = hidden/16.  Warp w works on slot
// w / ksplit, K part w % ksplit.  out[r] = bf16( bf16(sum_slot bf16(y_slot[r]) *
// wts[slot]) + addend[r] ); wts == NULL means weight 1 (single expert), addend
// may be NULL.  Mirrors expert_accum_k :399, round_bf16_k :404, add_k :248.
// ---------------------------------------------------------------------------
template <int BATCH>
__global__ void __launch_bounds__(kMaxWarps * 32)
    i4_down_kernel(const uint32_t *__restrict__ down_w, const uint16_t *__restrict__ down_s,
                   const uint16_t *__restrict__ mid, const int *__restrict__ slot_expert,
                   const float *__restrict__ wts, const uint16_t *__restrict__ addend, uint16_t *__restrict__ out,
                   int cols /*inter*/, int rows /*hidden*/, int slots, int ksplit, int nbatch) {
  extern __shared__ __align__(16) unsigned char smem[];
  __shared__ float partial[kMaxWarps][16];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t = lane & 3;
  const size_t stage_stride = i4_stage_bytes(cols, BATCH);
  for (int s = 0; s < slots; ++s) {
    I4Stage st = i4_stage_carve(smem + s * stage_stride, cols, BATCH);
    stage_x_i4(reinterpret_cast<const uint4 *>(mid + (size_t)s * cols), st, cols, BATCH, tid, blockDim.x);
  }
  __syncthreads();
  const int slot = warp / ksplit, kpart = warp - slot * ksplit;
  const int e = slot_expert ? slot_expert[slot] : slot;
  const int row0 = blockIdx.x * 16;
  const size_t wrow = cols / 32;
  const size_t ebase = (size_t)e * rows * wrow;
  I4Stage st = i4_stage_carve(smem + slot * stage_stride, cols, BATCH);
  const uint4 *w_lo = reinterpret_cast<const uint4 *>(down_w) + ebase + (size_t)(row0 + g) * wrow;
  const uint4 *w_hi = w_lo + 8 * wrow;
  const uint16_t *s_sel = down_s + ebase + (size_t)(row0 + g + 8 * (t >> 1)) * wrow + 2 * (t & 1);
  XFragLane xl = xfrag_lane(st, lane, BATCH);
  float acc = i4_rows16_accumulate<BATCH>(w_lo, w_hi, s_sel, xl, st.xsum, kpart * nbatch * BATCH, nbatch, lane);
  acc += __shfl_xor_sync(0xffffffffu, acc, 1);
  if ((t & 1) == 0) partial[warp][g + 8 * (t >> 1)] = acc;
  __syncthreads();
  if (tid < 16) {
    float o = 0.f;
    for (int s = 0; s < slots; ++s) {
      float ys = 0.f;
      for (int k = 0; k < ksplit; ++k) ys += partial[s * ksplit + k][tid];
      ys = round_bf16(ys);
      o = fmaf(ys, wts ? wts[s] : 1.0f, o);
    }
    o = round_bf16(o);
    if (addend) o = round_bf16(o + bf16_bits_to_f32(addend[row0 + tid]));
    out[row0 + tid] = f32_to_bf16_bits(o);
  }
}

__global__ void f32_to_bf16_kernel(const float *__restrict__ x, uint16_t *__restrict__ y, long n) {
  long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) y[i] = f32_to_bf16_bits(x[i]);
}

// ---------------------------------------------------------------------------
// host-side launch helpers
// ---------------------------------------------------------------------------
// Split `kblocks` k-blocks over warps: picks nwarps (<= max_warps, dividing
// kblocks) and a BATCH in {8,7,4,2,1} dividing the per-warp count.
struct KSplit {
  int nwarps, batch, nbatch;
};

static KSplit pick_split(int kblocks, int max_warps) {
  KSplit k{1, 1, kblocks};
  for (int nw = max_warps; nw >= 1; --nw)
    if (kblocks % nw == 0) {
      k.nwarps = nw;
      break;
    }
  int per = kblocks / k.nwarps;
  const int cand[5] = {8, 7, 4, 2, 1};
  for (int b : cand)
    if (per % b == 0) {
      k.batch = b;
      break;
    }
  k.nbatch = per / k.batch;
  return k;
}

#define BLOK_DISPATCH_BATCH(batch, ...)                        \
  switch (batch) {                                             \
    case 8: { constexpr int B = 8; __VA_ARGS__; } break;       \
    case 7: { constexpr int B = 7; __VA_ARGS__; } break;       \
    case 4: { constexpr int B = 4; __VA_ARGS__; } break;       \
    case 2: { constexpr int B = 2; __VA_ARGS__; } break;       \
    default: { constexpr int B = 1; __VA_ARGS__; } break;      \
  }

template <typename K>
static int ensure_smem(K kernel, size_t bytes) {
  if (bytes > 48 * 1024) BLOK_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes));
  return BLOK_OK;
}

int launch_i4_gemv16(const uint32_t *w, const uint16_t *scale, const uint16_t *x, uint16_t *y_bf16, float *y_f32,
                     int rows, int cols, cudaStream_t stream) {
  KSplit ks = pick_split(cols / 128, 8);
  size_t smem = i4_stage_bytes(cols, ks.batch);
  BLOK_DISPATCH_BATCH(ks.batch, {
    if (y_bf16) {
      int rc = ensure_smem(i4_gemv16_kernel<B, uint16_t>, smem);
      if (rc) return rc;
      i4_gemv16_kernel<B, uint16_t><<<rows / 16, ks.nwarps * 32, smem, stream>>>(w, scale, x, y_bf16, cols, ks.nbatch);
    } else {
      int rc = ensure_smem(i4_gemv16_kernel<B, float>, smem);
      if (rc) return rc;
      i4_gemv16_kernel<B, float><<<rows / 16, ks.nwarps * 32, smem, stream>>>(w, scale, x, y_f32, cols, ks.nbatch);
    }
  });
  return launch_status("i4_gemv16_kernel");
}

int launch_i4_gateup(const uint32_t *gate_w, const uint16_t *gate_s, const uint32_t *up_w, const uint16_t *up_s,
                     const uint16_t *x, const int *slot_expert, uint16_t *mid, int hidden, int inter, int slots,
                     cudaStream_t stream) {
  KSplit ks = pick_split(hidden / 128, 8);
  size_t smem = i4_stage_bytes(hidden, ks.batch);
  BLOK_DISPATCH_BATCH(ks.batch, {
    int rc = ensure_smem(i4_gateup_kernel<B>, smem);
    if (rc) return rc;
    i4_gateup_kernel<B><<<dim3(inter / 8, slots), ks.nwarps * 32, smem, stream>>>(gate_w, gate_s, up_w, up_s, x,
                                                                                   slot_expert, mid, hidden, inter,
                                                                                   ks.nbatch);
  });
  return launch_status("i4_gateup_kernel");
}

int launch_i4_down(const uint32_t *down_w, const uint16_t *down_s, const uint16_t *mid, const int *slot_expert,
                   const float *wts, const uint16_t *addend, uint16_t *out, int hidden, int inter, int slots,
                   cudaStream_t stream) {
  // warps = slots * ksplit <= 16
  int max_split = kMaxWarps / slots;
  if (max_split < 1) {
    set_error("i4_down: %d slots exceed %d warps", slots, kMaxWarps);
    return BLOK_ERR_SHAPE;
  }
  KSplit ks = pick_split(inter / 128, max_split > 8 ? 8 : max_split);
  size_t smem = i4_stage_bytes(inter, ks.batch) * slots;
  BLOK_DISPATCH_BATCH(ks.batch, {
    int rc = ensure_smem(i4_down_kernel<B>, smem);
    if (rc) return rc;
    i4_down_kernel<B><<<hidden / 16, slots * ks.nwarps * 32, smem, stream>>>(down_w, down_s, mid, slot_expert, wts,
                                                                             addend, out, inter, hidden, slots,
                                                                             ks.nwarps, ks.nbatch);
  });
  return launch_status("i4_down_kernel");
}

static bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

int launch_i4_gemv16_imma(const uint32_t *w, const uint16_t *scale, const uint16_t *x, uint16_t *y_bf16, float *y_f32, int rows,
                          int cols, cudaStream_t stream);

}  // namespace blok

using namespace blok;

extern "C" int blok_i4_dequant(const uint32_t *w, const blok_bf16_t *scale, blok_bf16_t *out, int rows, int cols,
                               blok_stream_t stream) {
  BLOK_REQUIRE(rows >= 0 && cols >= 0 && cols % 32 == 0, BLOK_ERR_SHAPE, "blok_i4_dequant: cols %d must be a multiple of 32", cols);
  if (rows == 0 || cols == 0) return BLOK_OK;  // empty tensors may carry null pointers
  BLOK_REQUIRE(w && scale && out, BLOK_ERR_ARG, "blok_i4_dequant: null pointer");
  BLOK_REQUIRE(aligned16(out), BLOK_ERR_ARG, "blok_i4_dequant: out must be 16-byte aligned");
  long words = (long)rows * (cols / 8);
  if (words == 0) return BLOK_OK;
  i4_dequant_kernel<<<(unsigned)((words + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
      w, scale, reinterpret_cast<uint4 *>(out), words, cols / 8);
  return launch_status("i4_dequant_kernel");
}

static int i4_gemv_common(const uint32_t *w, const blok_bf16_t *scale, const blok_bf16_t *x_bf16, const float *x_f32,
                          blok_bf16_t *y_bf16, float *y_f32, int rows, int cols, cudaStream_t stream) {
  BLOK_REQUIRE(rows >= 0 && cols > 0 && cols % 32 == 0, BLOK_ERR_SHAPE, "blok_i4_gemv: cols %d must be a positive multiple of 32", cols);
  if (rows == 0) return BLOK_OK;  // empty tensors may carry null pointers
  BLOK_REQUIRE(w && scale && (x_bf16 || x_f32) && (y_bf16 || y_f32), BLOK_ERR_ARG, "blok_i4_gemv: null pointer");
  BLOK_REQUIRE(aligned16(w), BLOK_ERR_ARG, "blok_i4_gemv: weight_packed must be 16-byte aligned");
  // BLOK_I4_GEMV_IMPL=imma (read at every call): the integer tensor-core consumer of i4_imma.cuh, an experiment in
  // cutting the unpack work; it keeps 14 bits below the largest activation of each 32-column group
  if (x_bf16 && rows % 16 == 0 && cols % 128 == 0 && aligned16(x_bf16) && cols <= 32768) {
    const char *impl = getenv("BLOK_I4_GEMV_IMPL");
    if (impl && strcmp(impl, "imma") == 0) return launch_i4_gemv16_imma(w, scale, x_bf16, y_bf16, y_f32, rows, cols, stream);
  }
  bool tc = x_bf16 && rows % 16 == 0 && cols % 256 == 0 && aligned16(x_bf16) && cols <= 32768;
  if (tc) return launch_i4_gemv16(w, scale, x_bf16, y_bf16, y_f32, rows, cols, stream);
  unsigned blocks = (unsigned)((rows + 7) / 8);
  if (x_bf16 && y_bf16) i4_gemv_scalar_kernel<uint16_t, uint16_t><<<blocks, 256, 0, stream>>>(w, scale, x_bf16, y_bf16, rows, cols);
  else if (x_bf16) i4_gemv_scalar_kernel<uint16_t, float><<<blocks, 256, 0, stream>>>(w, scale, x_bf16, y_f32, rows, cols);
  else if (y_bf16) i4_gemv_scalar_kernel<float, uint16_t><<<blocks, 256, 0, stream>>>(w, scale, x_f32, y_bf16, rows, cols);
  else i4_gemv_scalar_kernel<float, float><<<blocks, 256, 0, stream>>>(w, scale, x_f32, y_f32, rows, cols);
  return launch_status("i4_gemv_scalar_kernel");
}

extern "C" int blok_i4_gemv(const uint32_t *w, const blok_bf16_t *scale, const blok_bf16_t *x, blok_bf16_t *y, int rows,
                            int cols, blok_stream_t stream) {
  return i4_gemv_common(w, scale, x, nullptr, y, nullptr, rows, cols, (cudaStream_t)stream);
}

extern "C" int blok_i4_gemv_f32(const uint32_t *w, const blok_bf16_t *scale, const float *x, float *y, int rows,
                                int cols, blok_stream_t stream) {
  return i4_gemv_common(w, scale, nullptr, x, nullptr, y, rows, cols, (cudaStream_t)stream);
}

extern "C" size_t blok_expert_ffn_workspace_bytes(int hidden, int inter) {
  (void)hidden;
  return inter > 0 ? (size_t)inter * sizeof(uint16_t) : 0;
}

extern "C" int blok_expert_ffn(const uint32_t *gate_w, const blok_bf16_t *gate_s, const uint32_t *up_w,
                               const blok_bf16_t *up_s, const uint32_t *down_w, const blok_bf16_t *down_s,
                               const blok_bf16_t *x, blok_bf16_t *y, int hidden, int inter, void *workspace,
                               size_t workspace_bytes, blok_stream_t stream) {
  BLOK_REQUIRE(gate_w && gate_s && up_w && up_s && down_w && down_s && x && y && workspace, BLOK_ERR_ARG,
               "blok_expert_ffn: null pointer");
  BLOK_REQUIRE(hidden > 0 && inter > 0 && hidden % 256 == 0 && inter % 256 == 0 && hidden <= 32768 && inter <= 32768,
               BLOK_ERR_SHAPE, "blok_expert_ffn: hidden %d and inter %d must be multiples of 256 (<= 32768)", hidden, inter);
  BLOK_REQUIRE(workspace_bytes >= blok_expert_ffn_workspace_bytes(hidden, inter), BLOK_ERR_WORKSPACE,
               "blok_expert_ffn: workspace too small");
  BLOK_REQUIRE(aligned16(gate_w) && aligned16(up_w) && aligned16(down_w) && aligned16(x) && aligned16(workspace),
               BLOK_ERR_ARG, "blok_expert_ffn: pointers must be 16-byte aligned");
  uint16_t *mid = static_cast<uint16_t *>(workspace);
  int rc = launch_i4_gateup(gate_w, gate_s, up_w, up_s, x, nullptr, mid, hidden, inter, 1, (cudaStream_t)stream);
  if (rc) return rc;
  return launch_i4_down(down_w, down_s, mid, nullptr, nullptr, nullptr, y, hidden, inter, 1, (cudaStream_t)stream);
}

// ---------------------------------------------------------------------------
// blok_expert_ffn_static: the single-expert FFN for callers that must not allocate.
//
// Some hosts of this library cannot call cudaMalloc at the point where they run an
// expert: a serving loop that has handed all device memory to its own pool, code
// running inside a region where the allocator is locked, or a plugin boundary that
// forbids allocation after start-up.  blok_expert_ffn makes such a caller bring a
// workspace for the intermediate vector (mid = SiLU(gate x) * up x); this variant
// keeps that vector in a fixed array that is part of the library image instead.
//
// The array below lives in every CUDA context that loads the library, for as long
// as the context lives (BLOK_STATIC_MAX_INTER * 2 bytes = 16 KB per GPU).  In host
// code the name g_static_mid is only a handle for the symbol, not a device address:
// the address that kernels may use comes from cudaGetSymbolAddress, asked once per
// device with that device current, and cached.
// ---------------------------------------------------------------------------
static __device__ __align__(256) uint16_t g_static_mid[BLOK_STATIC_MAX_INTER];

namespace blok {
constexpr int kMaxDevices = 64;
static std::mutex g_static_mutex;
static uint16_t *g_static_mid_addr[kMaxDevices] = {};

// Device address of g_static_mid on the current device (looked up on first use).
static int static_mid_address(uint16_t **out) {
  int dev = 0;
  BLOK_CUDA(cudaGetDevice(&dev));
  BLOK_REQUIRE(dev >= 0 && dev < kMaxDevices, BLOK_ERR_STATE, "blok_expert_ffn_static: device ordinal %d not supported", dev);
  std::lock_guard<std::mutex> lock(g_static_mutex);
  if (!g_static_mid_addr[dev]) {
    void *p = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&p, g_static_mid);
    if (e != cudaSuccess) return cuda_fail(e, "cudaGetSymbolAddress(g_static_mid)");
    BLOK_REQUIRE(p != nullptr, BLOK_ERR_CUDA, "blok_expert_ffn_static: symbol address is null");
    g_static_mid_addr[dev] = static_cast<uint16_t *>(p);
  }
  *out = g_static_mid_addr[dev];
  return BLOK_OK;
}
}  // namespace blok

extern "C" int blok_expert_ffn_static_max_inter(void) { return BLOK_STATIC_MAX_INTER; }

extern "C" int blok_expert_ffn_static(const uint32_t *gate_w, const blok_bf16_t *gate_s, const uint32_t *up_w,
                                      const blok_bf16_t *up_s, const uint32_t *down_w, const blok_bf16_t *down_s,
                                      const blok_bf16_t *x, blok_bf16_t *y, int hidden, int inter,
                                      blok_stream_t stream) {
  BLOK_REQUIRE(gate_w && gate_s && up_w && up_s && down_w && down_s && x && y, BLOK_ERR_ARG,
               "blok_expert_ffn_static: null pointer");
  BLOK_REQUIRE(hidden > 0 && inter > 0 && hidden % 256 == 0 && inter % 256 == 0 && hidden <= 32768, BLOK_ERR_SHAPE,
               "blok_expert_ffn_static: hidden %d and inter %d must be positive multiples of 256 (hidden <= 32768)",
               hidden, inter);
  BLOK_REQUIRE(inter <= BLOK_STATIC_MAX_INTER, BLOK_ERR_WORKSPACE,
               "blok_expert_ffn_static: inter %d exceeds the built-in scratch of %d values; use blok_expert_ffn with a "
               "caller workspace",
               inter, BLOK_STATIC_MAX_INTER);
  BLOK_REQUIRE(aligned16(gate_w) && aligned16(up_w) && aligned16(down_w) && aligned16(x), BLOK_ERR_ARG,
               "blok_expert_ffn_static: pointers must be 16-byte aligned");
  uint16_t *mid = nullptr;
  int rc = static_mid_address(&mid);
  if (rc) return rc;
  // every element of mid[0, inter) is rewritten by the gate/up kernel before the down kernel reads it,
  // so nothing left over from an earlier call can leak into this one
  rc = launch_i4_gateup(gate_w, gate_s, up_w, up_s, x, nullptr, mid, hidden, inter, 1, (cudaStream_t)stream);
  if (rc) return rc;
  return launch_i4_down(down_w, down_s, mid, nullptr, nullptr, nullptr, y, hidden, inter, 1, (cudaStream_t)stream);
}
