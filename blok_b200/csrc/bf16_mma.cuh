// bf16 mat-vec building blocks on mma.sync tensor cores (see bf16_kernels.cu for the mapping).
#pragma once
#include "common.cuh"

namespace blok {

constexpr int kBfMaxWarps = 16;
constexpr int kBfBatch = 4;  // k-steps (uint4 pairs) in flight per lane

__host__ __device__ constexpr size_t bf16_x_row_bytes(int cols) { return (size_t)cols * 2 + 64; }

// Stage T (<= 8) activation rows into shared memory with a 64-byte skew per row.
__device__ __forceinline__ void stage_x_bf16(const uint16_t *x, unsigned char *smem, int cols, int T, int tid,
                                             int nthreads) {
  const int per_row = cols / 8;
  for (int u = tid; u < per_row * T; u += nthreads) {
    int tok = u / per_row, c = u - tok * per_row;
    uint4 v = reinterpret_cast<const uint4 *>(x + (size_t)tok * cols)[c];
    reinterpret_cast<uint4 *>(smem + tok * bf16_x_row_bytes(cols))[c] = v;
  }
}

// Accumulate k-steps [ks0, ks0 + nsteps) for this warp's 16 rows.
__device__ __forceinline__ void bf16_rows16_accumulate(const uint4 *__restrict__ w_lo, const uint4 *__restrict__ w_hi,
                                                       const uint4 *xrow /*token g row, +t applied*/, int ks0,
                                                       int nsteps, int t, float (&d)[4]) {
  int s = 0;
  for (; s + kBfBatch <= nsteps; s += kBfBatch) {
    uint4 wl[kBfBatch], wh[kBfBatch];
#pragma unroll
    for (int k = 0; k < kBfBatch; ++k) {
      wl[k] = ldg_stream(w_lo + (ks0 + s + k) * 4 + t);
      wh[k] = ldg_stream(w_hi + (ks0 + s + k) * 4 + t);
    }
#pragma unroll
    for (int k = 0; k < kBfBatch; ++k) {
      uint4 xb = xrow[(ks0 + s + k) * 4];
      mma_bf16_16816(d, wl[k].x, wh[k].x, wl[k].y, wh[k].y, xb.x, xb.y);
      mma_bf16_16816(d, wl[k].z, wh[k].z, wl[k].w, wh[k].w, xb.z, xb.w);
    }
  }
  for (; s < nsteps; ++s) {
    uint4 wl = ldg_stream(w_lo + (ks0 + s) * 4 + t);
    uint4 wh = ldg_stream(w_hi + (ks0 + s) * 4 + t);
    uint4 xb = xrow[(ks0 + s) * 4];
    mma_bf16_16816(d, wl.x, wh.x, wl.y, wh.y, xb.x, xb.y);
    mma_bf16_16816(d, wl.z, wh.z, wl.w, wh.w, xb.z, xb.w);
  }
}

template <int BATCH>
struct Bf16Batch {
  uint4 wl[BATCH], wh[BATCH];
};

template <int BATCH>
__device__ __forceinline__ void bf16_batch_load(Bf16Batch<BATCH> &b, const uint4 *__restrict__ w_lo,
                                                const uint4 *__restrict__ w_hi, int ks0, int t) {
#pragma unroll
  for (int k = 0; k < BATCH; ++k) {
    b.wl[k] = ldg_stream(w_lo + (ks0 + k) * 4 + t);
    b.wh[k] = ldg_stream(w_hi + (ks0 + k) * 4 + t);
  }
}

// xrow points at the activation segment (+t applied); ksx is the k-step index inside it.
template <int BATCH>
__device__ __forceinline__ void bf16_batch_compute(const Bf16Batch<BATCH> &b, const uint4 *xrow, int ksx,
                                                   float (&d)[4]) {
#pragma unroll
  for (int k = 0; k < BATCH; ++k) {
    uint4 xb = xrow[(ksx + k) * 4];
    mma_bf16_16816(d, b.wl[k].x, b.wh[k].x, b.wl[k].y, b.wh[k].y, xb.x, xb.y);
    mma_bf16_16816(d, b.wl[k].z, b.wh[k].z, b.wl[k].w, b.wh[k].w, xb.z, xb.w);
  }
}

}  // namespace blok
