// INT4 (pack_quantized, group 32) mat-vec on the INTEGER tensor-core path: an alternative consumer to i4_mma.cuh,
// selected with BLOK_I4_GEMV_IMPL=imma.  Same result contract as matvec_i4_bf16_scale_k (src/kimi_exec.cu:300-323)
// within the floating-point bar; it differs from i4_mma.cuh in where rounding happens, not in what is computed.
//
// Why: unpacking a nibble to a bf16 operand costs about one integer instruction per nibble pair plus shifts
// (~56 per 128-column k-block and lane); an 8-bit operand takes the nibble where it lies: byte = 16 (q + 8) is
// (w << 4) & 0xf0f0f0f0 for the even nibbles and w & 0xf0f0f0f0 for the odd ones, 3 instructions per 8 nibbles.
//
// The activations become block integers per scale group g of 32 columns: with E the largest exponent in the group,
//   X_c = round(x_c * 2^(13 - E))        |X_c| < 2^14, exact for every x_c within 2^-6 of the group's largest
//   X_c = 256 h_c + l_c                  h, l signed bytes (balanced split)
// so that  sum_c q_c x_c = 2^(E-13) / 16 * (256 D_h + D_l - 128 sum_c X_c),  D_limb = sum_c 16 (q_c + 8) limb_c,
// where D_h and D_l are exact int32 results of mma.m16n8k32 (u8 x s8).  Rounding x to an integer costs at most half a
// unit, 2^-14 of the group's largest value, per element: for activations within a few octaves of each other that is
// far below the bf16 rounding of the result (and below the reference's own bf16 rounding of every dequantised
// weight, :312), but a value more than 2^14 below the largest of its 32-column group is lost.  That limit is why
// this path is opt-in and the bf16-operand path stays the default.
//
// Mapping (as in i4_mma.cuh): a warp owns 16 weight rows, lane (g, t) loads one uint4 = scale group t of k-block kb
// of rows g and g + 8.  Word i of that uint4 feeds MMA i: a0/a1 = even nibbles of row g / g + 8 (k slots 4t..4t+3),
// a2/a3 = the odd nibbles (k slots 16+4t..).  B is block structured: column n = 2 t' + limb carries the limbs of
// quad-lane t' and zeros elsewhere, so D[row][2t + limb] is the limb sum of row over group t alone and lands in lane
// (g, t) itself: every lane post-scales its own group for both of its rows.
#pragma once
#include "common.cuh"

namespace blok {

constexpr uint32_t kByteNibMask = 0xf0f0f0f0u;

__device__ __forceinline__ void mma_u8s8_16832(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                               uint32_t b1) {
  asm("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Staged activations of `cols` columns (cols % 128 == 0):
//   xq    bytes [kb][t][limb][i][8]: the B registers (b0 = even columns, b1 = odd columns) of MMA i for quad-lane t
//   meta  [kb * 4 + t] = (f = 2^(E - 144) as float bits, off = 128 * sum X) per scale group
//   zero  what the non-supplying lanes read
struct ImmaStage {
  unsigned char *xq;
  uint2 *meta;
  uint4 *zero;
};

__host__ __device__ constexpr size_t imma_stage_bytes(int cols) {
  return (size_t)cols * 2 + (size_t)(cols / 32) * 8 + 128;
}

__device__ __forceinline__ ImmaStage imma_stage_carve(unsigned char *smem, int cols) {
  ImmaStage s;
  s.xq = smem;
  s.meta = reinterpret_cast<uint2 *>(smem + (size_t)cols * 2);
  s.zero = reinterpret_cast<uint4 *>(smem + (size_t)cols * 2 + (size_t)(cols / 32) * 8);
  return s;
}

// Quantises one unit (8 consecutive bf16 values = one packed word's columns, v as they lie in memory) of unit index u
// and stores its bytes; lane i == 0 of the group also stores the group's meta word.  The four units of a scale group
// must be in four ADJACENT, converged lanes (the group exponent and sum are exchanged with xor-shuffles 1 and 2);
// lanes with live == false take part in the shuffles and store nothing.
__device__ __forceinline__ void imma_stage_unit(const uint4 &v, int u, bool live, unsigned char *xq, uint2 *meta) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
  // biased exponent of the largest magnitude in the unit, then in the group
  uint32_t e = 0;
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    e = max(e, (w[k] >> 7) & 0xffu);
    e = max(e, (w[k] >> 23) & 0xffu);
  }
  e = max(e, __shfl_xor_sync(0xffffffffu, e, 1));
  e = max(e, __shfl_xor_sync(0xffffffffu, e, 2));
  // groups whose values are all below 2^-108 (or zero) contribute nothing; a NaN/Inf exponent is clamped
  const bool dead = e < 20u;
  e = min(e, 254u);
  const float up = __uint_as_float((267u - e) << 23);  // 2^(13 - (e - 127)) = 2^(140 - e)
  int sum = 0;
  uint32_t hb[2] = {0, 0}, lb[2] = {0, 0};  // [parity of the column] four bytes each
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    const float xv = (k & 1) ? bf16hi(w[k >> 1]) : bf16lo(w[k >> 1]);
    int X = dead ? 0 : __float2int_rn(xv * up);
    X = max(-16383, min(16383, X));
    sum += X;
    const int h = (X + 128) >> 8;
    const int l = X - h * 256;
    hb[k & 1] |= (uint32_t)(h & 0xff) << (8 * (k >> 1));
    lb[k & 1] |= (uint32_t)(l & 0xff) << (8 * (k >> 1));
  }
  sum += __shfl_xor_sync(0xffffffffu, sum, 1);
  sum += __shfl_xor_sync(0xffffffffu, sum, 2);
  if (live) {
    const int kb = u >> 4, t = (u >> 2) & 3, i = u & 3;
    unsigned char *base = xq + (size_t)kb * 256 + t * 64 + i * 8;
    *reinterpret_cast<uint2 *>(base) = make_uint2(hb[0], hb[1]);
    *reinterpret_cast<uint2 *>(base + 32) = make_uint2(lb[0], lb[1]);
    if (i == 0) meta[u >> 2] = make_uint2(dead ? 0u : (e - 17u) << 23, (uint32_t)(128 * sum));
  }
}

// Quantises x (bf16, global) to block integers in MMA order.  Called by all threads of the CTA (a multiple of 32).
__device__ __forceinline__ void stage_x_imma(const uint4 *x, const ImmaStage &st, int cols, int tid, int nthreads) {
  const int units = cols / 8;
  for (int u0 = 0; u0 < units; u0 += nthreads) {
    const int u = u0 + tid;
    const bool live = u < units;  // units is a multiple of 4, so a group's four lanes are live together
    imma_stage_unit(live ? x[u] : make_uint4(0, 0, 0, 0), u, live, st.xq, st.meta);
  }
  for (int u = tid; u < 8; u += nthreads) st.zero[u] = make_uint4(0, 0, 0, 0);
}

// Read-only per-lane view of the B operands: lanes with (g >> 1) == t supply limb (g & 1) of their quad-lane's group.
struct ImmaLane {
  const uint4 *ptr;  // two uint4 per k-block: MMAs 0,1 and 2,3
  int kb_stride;     // in uint4: 16 for supplying lanes, 0 for the others
};

__device__ __forceinline__ ImmaLane imma_lane(const ImmaStage &st, int lane) {
  const int g = lane >> 2, t = lane & 3;
  const bool supply = (g >> 1) == t;
  ImmaLane x;
  x.ptr = supply ? reinterpret_cast<const uint4 *>(st.xq + t * 64 + (g & 1) * 32) : st.zero + 4 + (lane & 1);
  x.kb_stride = supply ? 16 : 0;
  return x;
}

// One k-block: the limb sums of this lane's group for rows g (d[0], d[1]) and g + 8 (d[2], d[3]).
__device__ __forceinline__ void imma_kblock(const uint4 &wl, const uint4 &wh, const uint4 *xp, int (&d)[4]) {
  const uint4 x01 = xp[0], x23 = xp[1];
  mma_u8s8_16832(d, (wl.x << 4) & kByteNibMask, (wh.x << 4) & kByteNibMask, wl.x & kByteNibMask, wh.x & kByteNibMask, x01.x, x01.y);
  mma_u8s8_16832(d, (wl.y << 4) & kByteNibMask, (wh.y << 4) & kByteNibMask, wl.y & kByteNibMask, wh.y & kByteNibMask, x01.z, x01.w);
  mma_u8s8_16832(d, (wl.z << 4) & kByteNibMask, (wh.z << 4) & kByteNibMask, wl.z & kByteNibMask, wh.z & kByteNibMask, x23.x, x23.y);
  mma_u8s8_16832(d, (wl.w << 4) & kByteNibMask, (wh.w << 4) & kByteNibMask, wl.w & kByteNibMask, wh.w & kByteNibMask, x23.z, x23.w);
}

// acc_lo / acc_hi += scale * 2^(E-144) * (256 D_h + D_l - 128 sum X) for rows g and g + 8, group t of the k-block.
__device__ __forceinline__ void imma_post(const int (&d)[4], uint2 meta, float s_lo, float s_hi, float &acc_lo, float &acc_hi) {
  const float f = __uint_as_float(meta.x);
  const int off = (int)meta.y;
  const float v_lo = (float)(d[0] * 256 + d[1] - off) * f;
  const float v_hi = (float)(d[2] * 256 + d[3] - off) * f;
  acc_lo = fmaf(s_lo, v_lo, acc_lo);
  acc_hi = fmaf(s_hi, v_hi, acc_hi);
}

}  // namespace blok
