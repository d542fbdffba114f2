// Shared device/host helpers for the sm_100a kernels.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <cstdint>
#include <cstdio>

#include "../../include/blok_b200.h"

namespace blok {

// ---- error plumbing (host) -------------------------------------------------
void set_error(const char *fmt, ...);
int cuda_fail(cudaError_t e, const char *what);

#define BLOK_CUDA(call)                                        \
  do {                                                         \
    cudaError_t e_ = (call);                                   \
    if (e_ != cudaSuccess) return ::blok::cuda_fail(e_, #call); \
  } while (0)

#define BLOK_REQUIRE(cond, code, ...) \
  do {                                \
    if (!(cond)) {                    \
      ::blok::set_error(__VA_ARGS__); \
      return (code);                  \
    }                                 \
  } while (0)

void count_launch();
void count_launches(long long n);  // kernels replayed from a CUDA graph
long long launches_so_far();

inline int launch_status(const char *what) {
  count_launch();
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? BLOK_OK : cuda_fail(e, what);
}

int sm_count();

// ---- device helpers ----------------------------------------------------------
__device__ __forceinline__ float bf16_bits_to_f32(uint32_t h) { return __uint_as_float(h << 16); }
__device__ __forceinline__ float bf16lo(uint32_t pair) { return __uint_as_float(pair << 16); }
__device__ __forceinline__ float bf16hi(uint32_t pair) { return __uint_as_float(pair & 0xffff0000u); }

__device__ __forceinline__ uint16_t f32_to_bf16_bits(float f) {
  return __bfloat16_as_ushort(__float2bfloat16_rn(f));
}
__device__ __forceinline__ float round_bf16(float f) { return __bfloat162float(__float2bfloat16_rn(f)); }

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  return (uint32_t)f32_to_bf16_bits(lo) | ((uint32_t)f32_to_bf16_bits(hi) << 16);
}

// 128-bit streaming load of weights that are read exactly once per pass.
__device__ __forceinline__ uint4 ldg_stream(const uint4 *p) {
  uint4 v;
  asm("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}

// D(16x8, fp32) += A(16x16, bf16, row) * B(16x8, bf16, col).
__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                               uint32_t b0, uint32_t b1) {
  asm(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

__device__ __forceinline__ float silu_mul_f32(float g, float u) { return g / (1.0f + __expf(-g)) * u; }

}  // namespace blok
