// INT4 (pack_quantized, group 32) mat-vec building blocks on mma.sync tensor cores.
//
// A batch-1 INT4 GEMV at HBM rate cannot afford the ~3 CUDA-core instructions per
// nibble of the scalar form (unpack, convert, FMA): at 6.5 TB/s the SMs would have
// to retire more lane-instructions than they can issue.  Here the multiply-adds
// run on the tensor cores and the CUDA cores only unpack.
//
// Mapping.  One warp owns 16 weight rows ("A rows": lane group g = lane/4 owns
// row g of the low half and row g of the high half).  A k-block is 128 columns:
// lane t = lane%4 of every group loads one uint4 = one 32-column scale group of
// each of its two rows, so a quad reads 64 contiguous bytes per row.
//
// A nibble n (= q + 8) becomes the bf16 number 128 + n by OR-ing it into the
// mantissa of 0x4300; no subtraction is done on the weights.  Instead the
// contraction computes sum (128+n) x and the per-group sum of x (xsum) removes
// the offset afterwards: sum q x = sum (128+n) x - 136 * xsum.
//
// The contraction index of mma.m16n8k16 may be permuted freely as long as A and
// B agree.  Lane t's four k-slots of an mma hold four of ITS OWN nibbles, so the
// four lanes of a quad contribute four DIFFERENT scale groups to one mma.  To
// keep the groups apart (each needs its own scale), the B operand is block
// structured: column n of B carries the x values of quad-lane (n & 3) and zeros
// elsewhere.  D[row][n] is then the dot product of row with group (n & 3) alone,
// and each lane scales two group sums of one row after the k-block.
//
// x is staged in shared memory in fragment order by stage_x_i4(): for k-block
// kb, word i (0..3) of a lane's uint4, quad lane t:  xfrag[(kb*4 + i)*4 + t] =
// {x0,x4 | x1,x5 | x2,x6 | x3,x7} with x_j = x[kb*128 + t*32 + i*8 + j], matching
// the (n_j, n_{j+4}) pairs that one AND+OR extracts from a packed word.
#pragma once
#include "common.cuh"

namespace blok {

constexpr uint32_t kNibMask = 0x000f000fu;
constexpr uint32_t kNibMagic = 0x43004300u;  // bf16 128.0 in both halves
constexpr float kNibOffset = 136.0f;         // 128 (magic) + 8 (nibble bias)

// (shifted & mask) | magic as ONE three-input logic op.  Written as lop3 because the
// plain C expression was compiled into two logic instructions per pair, which doubled
// the load on the integer pipe, the busiest one in these kernels.
__device__ __forceinline__ uint32_t nib_pair(uint32_t shifted) {
  uint32_t r;
  asm("lop3.b32 %0, %1, %2, %3, 0xea;" : "=r"(r) : "r"(shifted), "r"(kNibMask), "r"(kNibMagic));
  return r;
}

// Per-lane read-only state for the x fragments.  Supplying lanes walk the
// fragment array (16 uint4 per k-block); the other lanes stay inside the zero
// region, which is as large as one batch of k-blocks, so every lane issues the
// same LDS with the same immediate offsets and no predicate.
struct XFragLane {
  const uint4 *ptr;  // supplying lanes: xfrag + t; others: zero region + t
  int kb_stride;     // in uint4 per k-block: 16 for supplying lanes, 0 for the others
};

// Bytes of shared memory needed to stage `cols` columns for a given BATCH.
__host__ __device__ constexpr size_t i4_stage_bytes(int cols, int batch) {
  return (size_t)cols * 2 /*xfrag*/ + (size_t)batch * 256 + 64 /*zero region*/ + (size_t)(cols / 32) * 4 /*xsum*/;
}

struct I4Stage {
  uint4 *xfrag;  // cols/8 uint4
  uint4 *zero;   // batch*16 + 4 uint4
  float *xsum;   // cols/32 floats
};

__device__ __forceinline__ I4Stage i4_stage_carve(unsigned char *smem, int cols, int batch) {
  I4Stage s;
  s.xfrag = reinterpret_cast<uint4 *>(smem);
  s.zero = s.xfrag + cols / 8;
  s.xsum = reinterpret_cast<float *>(s.zero + batch * 16 + 4);
  return s;
}

// Stage x (bf16, global, cols % 256 == 0) into fragment order, with group sums.
// Called by all threads of the CTA (nthreads % 32 == 0); caller syncs afterwards.
// CG = true reads through L2 (ld.global.cg): needed when x was written earlier in
// the same kernel by another CTA.
template <bool CG = false>
__device__ __forceinline__ void stage_x_i4(const uint4 *x, const I4Stage &st, int cols, int batch, int tid,
                                           int nthreads) {
  for (int u = tid; u < cols / 8; u += nthreads) {
    uint4 v = CG ? __ldcg(x + u) : x[u];
    int kb = u >> 4, t = (u >> 2) & 3, i = u & 3;
    uint4 o;
    o.x = __byte_perm(v.x, v.z, 0x5410);
    o.y = __byte_perm(v.x, v.z, 0x7632);
    o.z = __byte_perm(v.y, v.w, 0x5410);
    o.w = __byte_perm(v.y, v.w, 0x7632);
    st.xfrag[kb * 16 + i * 4 + t] = o;
    float s = ((bf16lo(v.x) + bf16hi(v.x)) + (bf16lo(v.y) + bf16hi(v.y))) +
              ((bf16lo(v.z) + bf16hi(v.z)) + (bf16lo(v.w) + bf16hi(v.w)));
    s += __shfl_xor_sync(0xffffffffu, s, 1);
    s += __shfl_xor_sync(0xffffffffu, s, 2);
    if ((u & 3) == 0) st.xsum[u >> 2] = s;
  }
  for (int u = tid; u < batch * 16 + 4; u += nthreads) st.zero[u] = make_uint4(0, 0, 0, 0);
}

__device__ __forceinline__ XFragLane xfrag_lane(const I4Stage &st, int lane, int batch) {
  int g = lane >> 2, t = lane & 3;
  bool supply = (t == (g & 3));
  XFragLane x;
  (void)batch;
  // The zero lanes read 64 bytes further into their region than the supplying lanes do into a k-block: the fragment
  // array is a multiple of 128 bytes long, so without the shift both would hit the same banks in every 8-lane phase.
  x.ptr = supply ? st.xfrag + t : st.zero + 4 + t;
  x.kb_stride = supply ? 16 : 0;
  return x;
}

// All four words of one k-block: d = per-group dot products (offset form).  One chain of eight dependent MMAs; two
// chains of four (four more registers and adds per k-block) measured the same.
__device__ __forceinline__ void i4_kblock_mma(const uint4 &wl, const uint4 &wh, const uint4 *xp, float (&d)[4]) {
  const uint32_t al[4] = {wl.x, wl.y, wl.z, wl.w};
  const uint32_t ah[4] = {wh.x, wh.y, wh.z, wh.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    uint4 xb = xp[i * 4];
    uint32_t a = al[i], b = ah[i];
    mma_bf16_16816(d, nib_pair(a), nib_pair(b), nib_pair(a >> 4), nib_pair(b >> 4), xb.x, xb.y);
    mma_bf16_16816(d, nib_pair(a >> 8), nib_pair(b >> 8), nib_pair(a >> 12), nib_pair(b >> 12), xb.z, xb.w);
  }
}

// Accumulate NB = nbatch*BATCH k-blocks starting at k-block kb0 for this warp's 16
// A rows.  w_lo / w_hi point at the lane's own rows (uint4 units, row start);
// s_sel points at the scale row this lane post-scales (low row for t < 2, high
// row for t >= 2), already offset by j0 = 2*(t&1).  Returns the lane's partial
// sum for A row g + 8*(t>>1) over groups {j0, j0+1} of every k-block; the caller
// adds the partner lane (xor 1).
template <int BATCH>
__device__ __forceinline__ float i4_rows16_accumulate(const uint4 *__restrict__ w_lo, const uint4 *__restrict__ w_hi,
                                                      const uint16_t *__restrict__ s_sel, const XFragLane &xl,
                                                      const float *xsum, int kb0, int nbatch, int lane) {
  const int t = lane & 3;
  const bool hi_row = (t >> 1) != 0;
  const int j0 = 2 * (t & 1);
  float acc = 0.f;
  for (int b = 0; b < nbatch; ++b) {
    const int kbb = kb0 + b * BATCH;
    uint4 wl[BATCH], wh[BATCH];
    uint32_t sc[BATCH];
#pragma unroll
    for (int k = 0; k < BATCH; ++k) {
      wl[k] = ldg_stream(w_lo + (kbb + k) * 4 + t);
      wh[k] = ldg_stream(w_hi + (kbb + k) * 4 + t);
    }
#pragma unroll
    for (int k = 0; k < BATCH; ++k) sc[k] = __ldg(reinterpret_cast<const uint32_t *>(s_sel + (kbb + k) * 4));
    const uint4 *xp = xl.ptr + kbb * xl.kb_stride;
#pragma unroll
    for (int k = 0; k < BATCH; ++k) {
      float d[4] = {0.f, 0.f, 0.f, 0.f};
      i4_kblock_mma(wl[k], wh[k], xp + k * 16, d);
      float2 xs = *reinterpret_cast<const float2 *>(xsum + (kbb + k) * 4 + j0);
      float da = hi_row ? d[2] : d[0];
      float db = hi_row ? d[3] : d[1];
      acc = fmaf(bf16lo(sc[k]), fmaf(-kNibOffset, xs.x, da), acc);
      acc = fmaf(bf16hi(sc[k]), fmaf(-kNibOffset, xs.y, db), acc);
    }
  }
  return acc;
}

// Loads and arithmetic of one batch of k-blocks as separate steps, so that a caller
// can put the weight loads in flight, wait for something else (another CTA's
// results, say) and only then touch the activations.
template <int BATCH>
struct I4Batch {
  uint4 wl[BATCH], wh[BATCH];
  uint32_t sc[BATCH];
};

template <int BATCH>
__device__ __forceinline__ void i4_batch_load(I4Batch<BATCH> &b, const uint4 *__restrict__ w_lo,
                                              const uint4 *__restrict__ w_hi, const uint16_t *__restrict__ s_sel,
                                              int kb0, int t) {
#pragma unroll
  for (int k = 0; k < BATCH; ++k) {
    b.wl[k] = ldg_stream(w_lo + (kb0 + k) * 4 + t);
    b.wh[k] = ldg_stream(w_hi + (kb0 + k) * 4 + t);
  }
#pragma unroll
  for (int k = 0; k < BATCH; ++k) b.sc[k] = __ldg(reinterpret_cast<const uint32_t *>(s_sel + (kb0 + k) * 4));
}

// kbx is the k-block index of the batch inside the staged activation segment.
template <int BATCH>
__device__ __forceinline__ float i4_batch_compute(const I4Batch<BATCH> &b, const XFragLane &xl, const float *xsum,
                                                  int kbx, int lane, float acc) {
  const int t = lane & 3;
  const bool hi_row = (t >> 1) != 0;
  const int j0 = 2 * (t & 1);
  const uint4 *xp = xl.ptr + kbx * xl.kb_stride;
#pragma unroll
  for (int k = 0; k < BATCH; ++k) {
    float d[4] = {0.f, 0.f, 0.f, 0.f};
    i4_kblock_mma(b.wl[k], b.wh[k], xp + k * 16, d);
    float2 xs = *reinterpret_cast<const float2 *>(xsum + (kbx + k) * 4 + j0);
    float da = hi_row ? d[2] : d[0];
    float db = hi_row ? d[3] : d[1];
    acc = fmaf(bf16lo(b.sc[k]), fmaf(-kNibOffset, xs.x, da), acc);
    acc = fmaf(bf16hi(b.sc[k]), fmaf(-kNibOffset, xs.y, db), acc);
  }
  return acc;
}

// The same over an arbitrary k-block range [kb0, kb0 + nkb): full batches, then singles.
template <int BATCH>
__device__ __forceinline__ float i4_rows16_range(const uint4 *__restrict__ w_lo, const uint4 *__restrict__ w_hi,
                                                 const uint16_t *__restrict__ s_sel, const XFragLane &xl,
                                                 const float *xsum, int kb0, int nkb, int lane) {
  const int nfull = nkb / BATCH;
  float acc = i4_rows16_accumulate<BATCH>(w_lo, w_hi, s_sel, xl, xsum, kb0, nfull, lane);
  const int done = nfull * BATCH;
  if (done < nkb) acc += i4_rows16_accumulate<1>(w_lo, w_hi, s_sel, xl, xsum, kb0 + done, nkb - done, lane);
  return acc;
}

}  // namespace blok
