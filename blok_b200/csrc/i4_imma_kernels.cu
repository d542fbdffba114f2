// INT4 mat-vec through the integer tensor-core path (i4_imma.cuh): the same entry contract as the bf16-operand
// kernel of i4_kernels.cu (matvec_i4_slice, src/kimi_exec.cu:688-690), selected with BLOK_I4_GEMV_IMPL=imma.
#include "i4_imma.cuh"

namespace blok {

constexpr int kImmaMaxWarps = 8;
constexpr int kImmaBatch = 4;  // k-blocks whose weight loads are in flight per lane

// CTA = 16 rows, warps split the k-blocks.  y bf16 (YT = uint16_t) or bf16-valued fp32 (YT = float).
template <typename YT>
__global__ void __launch_bounds__(kImmaMaxWarps * 32)
    i4_gemv16_imma_kernel(const uint32_t *__restrict__ w, const uint16_t *__restrict__ scale, const uint16_t *__restrict__ x,
                          YT *__restrict__ y, int cols, int kb_per_warp) {
  extern __shared__ __align__(16) unsigned char smem[];
  __shared__ float partial[kImmaMaxWarps][16];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarps = blockDim.x >> 5;
  const int g = lane >> 2, t = lane & 3;
  const ImmaStage st = imma_stage_carve(smem, cols);
  stage_x_imma(reinterpret_cast<const uint4 *>(x), st, cols, tid, blockDim.x);
  __syncthreads();
  const int row0 = blockIdx.x * 16;
  const size_t wrow = cols / 32;  // uint4 per weight row == scales per scale row
  const uint4 *w_lo = reinterpret_cast<const uint4 *>(w) + (size_t)(row0 + g) * wrow + t;
  const uint4 *w_hi = w_lo + 8 * wrow;
  const uint16_t *s_lo = scale + (size_t)(row0 + g) * wrow + t;
  const uint16_t *s_hi = s_lo + 8 * wrow;
  const ImmaLane xl = imma_lane(st, lane);
  float acc_lo = 0.f, acc_hi = 0.f;
  const int kb_end = (warp + 1) * kb_per_warp;
  for (int kb0 = warp * kb_per_warp; kb0 < kb_end; kb0 += kImmaBatch) {
    uint4 wl[kImmaBatch], wh[kImmaBatch];
    uint16_t sl[kImmaBatch], sh[kImmaBatch];
#pragma unroll
    for (int k = 0; k < kImmaBatch; ++k) {
      const int kb = min(kb0 + k, kb_end - 1);  // a short last batch repeats its last k-block and skips it below
      wl[k] = ldg_stream(w_lo + (size_t)kb * 4);
      wh[k] = ldg_stream(w_hi + (size_t)kb * 4);
      sl[k] = __ldg(s_lo + (size_t)kb * 4);
      sh[k] = __ldg(s_hi + (size_t)kb * 4);
    }
#pragma unroll
    for (int k = 0; k < kImmaBatch; ++k) {
      const int kb = kb0 + k;
      if (kb < kb_end) {
        int d[4] = {0, 0, 0, 0};
        imma_kblock(wl[k], wh[k], xl.ptr + (size_t)kb * xl.kb_stride, d);
        imma_post(d, st.meta[kb * 4 + t], bf16_bits_to_f32(sl[k]), bf16_bits_to_f32(sh[k]), acc_lo, acc_hi);
      }
    }
  }
  // a row's four scale groups of every k-block sit in the four lanes of its quad
  acc_lo += __shfl_xor_sync(0xffffffffu, acc_lo, 1);
  acc_lo += __shfl_xor_sync(0xffffffffu, acc_lo, 2);
  acc_hi += __shfl_xor_sync(0xffffffffu, acc_hi, 1);
  acc_hi += __shfl_xor_sync(0xffffffffu, acc_hi, 2);
  if (t == 0) {
    partial[warp][g] = acc_lo;
    partial[warp][g + 8] = acc_hi;
  }
  __syncthreads();
  if (tid < 16) {
    float v = 0.f;
    for (int wi = 0; wi < nwarps; ++wi) v += partial[wi][tid];
    if constexpr (sizeof(YT) == 2) y[row0 + tid] = f32_to_bf16_bits(v);
    else y[row0 + tid] = round_bf16(v);
  }
}

// rows % 16 == 0, cols % 128 == 0, cols <= 32768, x 16-byte aligned.
int launch_i4_gemv16_imma(const uint32_t *w, const uint16_t *scale, const uint16_t *x, uint16_t *y_bf16, float *y_f32, int rows,
                          int cols, cudaStream_t stream) {
  const int kblocks = cols / 128;
  int nwarps = 1;
  for (int nw = kImmaMaxWarps; nw >= 1; --nw)
    if (kblocks % nw == 0) {
      nwarps = nw;
      break;
    }
  const size_t smem = imma_stage_bytes(cols);
  if (y_bf16) {
    if (smem > 48 * 1024)
      BLOK_CUDA(cudaFuncSetAttribute(i4_gemv16_imma_kernel<uint16_t>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    i4_gemv16_imma_kernel<uint16_t><<<rows / 16, nwarps * 32, smem, stream>>>(w, scale, x, y_bf16, cols, kblocks / nwarps);
  } else {
    if (smem > 48 * 1024)
      BLOK_CUDA(cudaFuncSetAttribute(i4_gemv16_imma_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    i4_gemv16_imma_kernel<float><<<rows / 16, nwarps * 32, smem, stream>>>(w, scale, x, y_f32, cols, kblocks / nwarps);
  }
  return launch_status("i4_gemv16_imma_kernel");
}

}  // namespace blok
