// Batch-1 routed-MoE decode layer as ONE persistent cooperative kernel.
// Reference: the MoE branch of the layer body, src/kimi_exec.cu:836-875.
//
// The layer is a chain of mat-vecs that together read 292 MB of weights exactly
// once, so the only thing that matters is keeping HBM busy from the first to the
// last byte.  One CTA per SM stays resident.  All work is cut into chunks of a few
// KB of weights (16 weight rows x a fixed k-range) that sit in ONE global queue in
// dependency order; every warp of the grid pulls chunk after chunk from the queue
// with an atomic counter, so the load balances itself and nothing waits at a
// phase boundary except where the data really is not there yet:
//
//   R   router logits, bf16               16 rows x 28 k-steps per chunk
//   A   shared-expert gate/up, bf16       (8 gate + 8 up rows) x 28 k-steps
//   B   the selected experts' INT4 gate/up (8 + 8 rows) x 14 k-blocks; needs the routing
//   C1  INT4 down, one (slot, 16 output rows) block per chunk; needs that slot's mid values
//   C2  shared-expert down, bf16          16 rows x 32 k-steps; needs the shared mid
//
// A chunk covers a row-block only partly.  Its 16 partial dot products go to a
// scratch slot indexed by the chunk's position in the row-block.  The warp that holds
// the LAST chunk of a row-block in queue order is its finisher: it sums the slots in
// index order and runs the row-block's epilogue: logits; SiLU*up -> mid; or, for the
// shared-expert down rows, the weighted combine of all nine contributions
//   y = bf16(bf16(sum_k w_k * bf16(y_k)) + bf16(shared)).
// Which warp computes a chunk varies from run to run; what is summed in which
// order does not, so results are deterministic.
//
// Everything one warp hands to another (partial sums, logits, mid values, per-slot
// outputs) travels as an 8-byte (value, tag) pair written with one store; the tag is
// the launch's epoch.  A reader polls a slot until the tag matches, so there is no
// fence, no arrival counter and no grid barrier: a down-projection chunk only waits
// if the very mid values it needs are not written yet, and its weight loads are in
// flight before it looks.  The routing is computed once per CTA from the tagged
// logits.  Every poll is bounded and records an error word read by
// blok_moe_layer_check; the launch is cooperative (all CTAs resident), so the warps
// being waited for are always running.  Weights stream through a warp-private
// cp.async ring in shared memory (each lane copies and later reads back its own
// words, so the ring needs no barrier).
#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <vector>

#include "bf16_mma.cuh"
#include "i4_mma.cuh"
#include "moe_layer.h"
#include "router_topk.cuh"

namespace blok {

#ifndef BLOK_FUSED_WARPS
#define BLOK_FUSED_WARPS 16
#endif
#ifndef BLOK_RING_DEPTH
#define BLOK_RING_DEPTH 5
#endif
constexpr int kMetaBytes = 4;  // per scale group: the sum of x

constexpr int kFusedWarps = BLOK_FUSED_WARPS;
constexpr int kFusedThreads = kFusedWarps * 32;
constexpr unsigned kSpinLimit = 1u << 22;  // polls before a wait gives up with an error word

enum { CTRL_QUEUE = 0, CTRL_EXIT = 4, CTRL_ERROR = 5, CTRL_EPOCH = 6 };  // word indices in the control block
constexpr int kTraceSlots = 16;

struct FusedParams {
  int hidden, inter, experts, topk, shared_inter;
  float routed_scale;
  const uint16_t *router_w;
  const float *router_bias;
  const uint32_t *gate_w, *up_w, *down_w;
  const uint16_t *gate_s, *up_s, *down_s;
  const uint16_t *shared_gate, *shared_up, *shared_down;
  const uint16_t *x;
  uint16_t *y;
  uint16_t *ids_out;
  float *wts_out;
  uint2 *logits;   // [experts] (router logit, launch tag)
  uint2 *mid;      // [topk + 1][mid_stride / 2] (two bf16 mid values, launch tag); row topk is the shared expert's
  int mid_stride;
  uint2 *ys;       // [topk + 1][hidden] (bf16-valued per-slot down output, launch tag)
  uint2 *partR, *partA, *partB, *partC2;  // [row-block][chunk][16] (partial dot product, launch tag)
  // chunking: steps per row-block, steps per chunk, chunks per row-block
  int sprR, spcR, cprR;
  int sprA, spcA, cprA;
  int sprB, spcB, cprB;
  int sprC1;
  int sprC2, spcC2, cprC2;
  unsigned cA0, cB0, cC10, cC20, total;  // first queue index of each phase; queue length
  unsigned *ctrl;
  long long *trace;  // optional: [0..15] launch-wide stamps, then [grid][kTraceSlots] per-CTA stamps (ns)
};

__device__ __forceinline__ long long global_ns() {
  long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ void trace_cta(const FusedParams &p, int slot) {
  if (p.trace) p.trace[16 + (size_t)blockIdx.x * kTraceSlots + slot] = global_ns();
}
__device__ __forceinline__ void trace_launch(const FusedParams &p, int slot) {
  if (p.trace) p.trace[slot] = global_ns();
}

// Results that one warp hands to another travel as (value, tag) pairs written with one
// 8-byte store; the tag is the launch's epoch, so a reader that polls a slot until the
// tag matches knows the value is this launch's, without any fence or counter.
__device__ __forceinline__ void st_tagged(uint2 *p, float v, unsigned tag) {
  asm volatile("st.global.cg.v2.u32 [%0], {%1, %2};" ::"l"(p), "r"(__float_as_uint(v)), "r"(tag) : "memory");
}
__device__ __forceinline__ float ld_tagged(const uint2 *p, unsigned tag, unsigned *err) {
  unsigned v, tg, it = 0;
  for (;;) {
    asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];" : "=r"(v), "=r"(tg) : "l"(p) : "memory");
    if (tg == tag) break;
    if (++it > kSpinLimit) {
      atomicExch(err, 3u);
      break;
    }
    __nanosleep(20);
  }
  return __uint_as_float(v);
}
// N tagged values at p[0], p[stride], ...: all loads are issued before any tag is looked at,
// so the wait is one memory round trip, not N; the batch is re-read only while a tag is missing.
template <int N>
__device__ __noinline__ void ld_tagged_n(const uint2 *p, int stride, int n, unsigned tag, unsigned *err,
                                            float (&out)[N]) {
  unsigned v[N], tg[N];
  for (unsigned it = 0;; ++it) {
#pragma unroll
    for (int i = 0; i < N; ++i)
      if (i < n) asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];" : "=r"(v[i]), "=r"(tg[i]) : "l"(p + (size_t)i * stride) : "memory");
    bool ok = true;
#pragma unroll
    for (int i = 0; i < N; ++i)
      if (i < n && tg[i] != tag) ok = false;
    if (ok) break;
    if (it > kSpinLimit) {
      atomicExch(err, 3u);
      break;
    }
    __nanosleep(20);
  }
#pragma unroll
  for (int i = 0; i < N; ++i) out[i] = i < n ? __uint_as_float(v[i]) : 0.f;
}

__device__ __forceinline__ float swiglu_ref_rounding(float g, float u) {
  // src/kimi_exec.cu:322 rounds both mat-vec outputs, :255 rounds SiLU and the product
  g = round_bf16(g);
  u = round_bf16(u);
  return round_bf16(round_bf16(g / (1.0f + expf(-g))) * u);
}

// ---- warp-private asynchronous weight ring ------------------------------------------
// Each lane copies its own weight words global -> shared with cp.async and reads
// the same words back later, so the ring is a FIFO extension of the lane's
// registers: no other lane touches a lane's words, and no barrier is needed.  One
// commit group per step, always (empty groups keep the count uniform), so
// "wait until at most kRingDepth-1 groups are pending" means "step s has landed".
//
// The scales of an INT4 chunk (8 bytes per row and k-block) are NOT fetched step by step: eight bytes per row per
// step touch a new 32-byte sector in 16 rows every step and fetch every sector four times over, which alone held the
// stream of weights + scales to 4.3-5.8 TB/s against 6.7 TB/s for the weights alone (measured with a trivial consumer).
// They are staged whole when the chunk's first weights are requested: consecutive lanes copy consecutive 8-byte pieces
// of a row, so a row's scales travel as full lines, once.
constexpr int kRingDepth = BLOK_RING_DEPTH;
constexpr int kRingStepBytes = 2 * 512;                  // low rows, high rows
constexpr int kScaleMaxSteps = 16;                       // k-blocks an INT4 chunk may have
constexpr int kScaleRowBytes = kScaleMaxSteps * 8 + 8;   // 136: the odd multiple of 8 spreads the 16 rows over all banks
constexpr int kScaleStageBytes = 16 * kScaleRowBytes;
constexpr int kWarpRingBytes = kRingDepth * kRingStepBytes + kScaleStageBytes;

__device__ __forceinline__ void cp_async16(uint32_t dst, const void *src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async8(uint32_t dst, const void *src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

enum { KIND_NONE = -1, KIND_R = 0, KIND_A = 1, KIND_B = 2, KIND_C1 = 3, KIND_C2 = 4 };

struct Chunk {
  int kind;
  int rb, kc;   // row-block inside its phase, chunk inside the row-block
  int k0, n;    // first step and number of steps
  int slot;     // routed slot (B, C1); topk for the shared expert
  const uint4 *w_lo, *w_hi;  // the lane's two weight rows (row start, uint4 units)
  const uint16_t *s_lo, *s_hi;  // INT4 kinds: scale rows of A rows 0..7 and 8..15 (row start)
  int s_stride;                 // elements between consecutive scale rows
};

__device__ __forceinline__ bool kind_is_i4(int kind) { return kind == KIND_B || kind == KIND_C1; }

__device__ __forceinline__ void ring_issue(const Chunk &ch, int s, uint32_t ring, int lane) {
  if (s < ch.n) {
    const int t = lane & 3;
    const uint32_t base = ring + (uint32_t)(s % kRingDepth) * kRingStepBytes + (uint32_t)lane * 16;
    cp_async16(base, ch.w_lo + (size_t)(ch.k0 + s) * 4 + t);
    cp_async16(base + 512, ch.w_hi + (size_t)(ch.k0 + s) * 4 + t);
  }
  cp_async_commit();
}

// The chunk's scales, whole: 16 rows x n k-blocks x 8 bytes, into the warp's scale stage (behind the ring).
__device__ __forceinline__ void scale_issue(const Chunk &ch, uint32_t ring, int lane) {
  const uint32_t stage = ring + kRingDepth * kRingStepBytes;
  const int pieces = 16 * ch.n;
  for (int pc = lane; pc < pieces; pc += 32) {
    const int row = pc / ch.n, s = pc - row * ch.n;
    const uint16_t *src = ((row & 8) ? ch.s_hi : ch.s_lo) + (size_t)(row & 7) * ch.s_stride + (size_t)(ch.k0 + s) * 4;
    cp_async8(stage + (uint32_t)(row * kScaleRowBytes + s * 8), src);
  }
}

__device__ __forceinline__ void ring_prologue(const Chunk &ch, uint32_t ring, int lane) {
  __syncwarp();  // every lane is done with the previous chunk's scales
  if (kind_is_i4(ch.kind)) scale_issue(ch, ring, lane);  // joins the first step's commit group
#pragma unroll
  for (int i = 0; i < kRingDepth; ++i) ring_issue(ch, i, ring, lane);
}

// Consumes the chunk's steps from the ring (issuing the steps beyond the prologue
// as slots free up) and returns the chunk's partial dot product for A row
// g + 8*(t>>1).  xfrag/xsum (INT4) or xrow (bf16) address the activation segment,
// whose first step is kx0.
__device__ __forceinline__ float ring_consume(const Chunk &ch, uint32_t ring, const unsigned char *ring_ptr,
                                              const XFragLane &xl, const float *xsum, const uint4 *xrow, int kx0,
                                              int lane) {
  const int t = lane & 3;
  const bool hi_row = (t >> 1) != 0;
  const int j0 = 2 * (t & 1);
  float acc = 0.f;
  float d[4] = {0.f, 0.f, 0.f, 0.f};
  const bool i4 = kind_is_i4(ch.kind);
  // this lane post-scales groups (j0, j0 + 1) of A row g + 8 * (t >> 1)
  const unsigned char *sc_lane = ring_ptr + kRingDepth * kRingStepBytes + ((lane >> 2) + 8 * (t >> 1)) * kScaleRowBytes + (t & 1) * 4;
  for (int s = 0; s < ch.n; ++s) {
    cp_async_wait<kRingDepth - 1>();
    if (s == 0) __syncwarp();  // the scales were copied by other lanes: their first group has landed as well
    const unsigned char *slotp = ring_ptr + (size_t)(s % kRingDepth) * kRingStepBytes;
    const uint4 wl = *reinterpret_cast<const uint4 *>(slotp + lane * 16);
    const uint4 wh = *reinterpret_cast<const uint4 *>(slotp + 512 + lane * 16);
    const int kx = ch.k0 - kx0 + s;
    if (i4) {
      const uint32_t sc = *reinterpret_cast<const uint32_t *>(sc_lane + s * 8);
      float dd[4] = {0.f, 0.f, 0.f, 0.f};
      i4_kblock_mma(wl, wh, xl.ptr + kx * xl.kb_stride, dd);
      const float2 xs = *reinterpret_cast<const float2 *>(xsum + kx * 4 + j0);
      const float da = hi_row ? dd[2] : dd[0];
      const float db = hi_row ? dd[3] : dd[1];
      acc = fmaf(bf16lo(sc), fmaf(-kNibOffset, xs.x, da), acc);
      acc = fmaf(bf16hi(sc), fmaf(-kNibOffset, xs.y, db), acc);
    } else {
      const uint4 xb = xrow[kx * 4];
      mma_bf16_16816(d, wl.x, wh.x, wl.y, wh.y, xb.x, xb.y);
      mma_bf16_16816(d, wl.z, wh.z, wl.w, wh.w, xb.z, xb.w);
    }
    ring_issue(ch, s + kRingDepth, ring, lane);
  }
  if (i4) {
    acc += __shfl_xor_sync(0xffffffffu, acc, 1);
    return acc;
  }
  return (t & 2) ? d[2] : d[0];
}

// Up to NU tagged 32-byte units (8 mid values each) at p, p + stride, ...: loads first, tags after.
template <int NU>
__device__ __forceinline__ void ld_tagged_units(const uint2 *p, int stride, int n, unsigned tag, unsigned *err,
                                                uint4 (&out)[NU]) {
  unsigned r[NU][8];
  for (unsigned it = 0;; ++it) {
#pragma unroll
    for (int i = 0; i < NU; ++i)
      if (i < n) {
        const uint2 *q = p + (size_t)i * stride;
        asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(r[i][0]), "=r"(r[i][1]), "=r"(r[i][2]), "=r"(r[i][3]) : "l"(q) : "memory");
        asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(r[i][4]), "=r"(r[i][5]), "=r"(r[i][6]), "=r"(r[i][7]) : "l"(q + 2) : "memory");
      }
    bool ok = true;
#pragma unroll
    for (int i = 0; i < NU; ++i)
      if (i < n && (r[i][1] != tag || r[i][3] != tag || r[i][5] != tag || r[i][7] != tag)) ok = false;
    if (ok) break;
    if (it > kSpinLimit) {
      atomicExch(err, 4u);
      break;
    }
    __nanosleep(20);
  }
#pragma unroll
  for (int i = 0; i < NU; ++i) out[i] = make_uint4(r[i][0], r[i][2], r[i][4], r[i][6]);
}

// Partial sums a finisher requests per round trip when it collects a row-block, and tagged 32-byte units a lane
// requests per round trip when it stages mid values (8 and 4 were measured slower: they spill).
constexpr int kCollect = 4;
constexpr int kStageUnits = 2;

// One warp stages `cols` mid values (tagged pairs written earlier in this launch by other
// warps; values that are not there yet are polled) into INT4 fragment order with group sums.
__device__ __noinline__ void warp_stage_i4(const uint2 *src, uint4 *xfrag, float *xsum, int cols, int lane,
                                              unsigned epoch, unsigned *err) {
  const int units = cols / 8;  // 32-byte tagged units; lane handles units lane, lane + 32, ...
  // kStageUnits units per lane are requested before any tag is looked at: one L2 round trip per kStageUnits * 32 units
  for (int u0 = lane; u0 < units; u0 += 32 * kStageUnits) {
    uint4 vv[kStageUnits];
    const int n = min(kStageUnits, (units - u0 + 31) / 32);
    ld_tagged_units<kStageUnits>(src + (size_t)u0 * 4, 32 * 4, n, epoch, err, vv);
#pragma unroll
    for (int j = 0; j < kStageUnits; ++j) {
      const int u = u0 + 32 * j;
      if (u < units) {  // units is a multiple of 32, so this is warp-uniform
        const uint4 v = vv[j];
        int kb = u >> 4, t = (u >> 2) & 3, i = u & 3;
        uint4 o;
        o.x = __byte_perm(v.x, v.z, 0x5410);
        o.y = __byte_perm(v.x, v.z, 0x7632);
        o.z = __byte_perm(v.y, v.w, 0x5410);
        o.w = __byte_perm(v.y, v.w, 0x7632);
        xfrag[kb * 16 + i * 4 + t] = o;
        float s = ((bf16lo(v.x) + bf16hi(v.x)) + (bf16lo(v.y) + bf16hi(v.y))) +
                  ((bf16lo(v.z) + bf16hi(v.z)) + (bf16lo(v.w) + bf16hi(v.w)));
        s += __shfl_xor_sync(0xffffffffu, s, 1);
        s += __shfl_xor_sync(0xffffffffu, s, 2);
        if ((u & 3) == 0) xsum[u >> 2] = s;
      }
    }
  }
  __syncwarp();
}

__global__ void __launch_bounds__(kFusedThreads, 1) moe_decode_fused_kernel(const FusedParams p) {
  extern __shared__ __align__(16) unsigned char smem[];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t = lane & 3;

  // ---- shared memory carve-up -------------------------------------------------
  unsigned char *sp = smem;
  uint4 *xnat = reinterpret_cast<uint4 *>(sp);  // x, natural order (bf16 operand)
  sp += (size_t)p.hidden * 2;
  uint4 *xfrag = reinterpret_cast<uint4 *>(sp);  // x, INT4 fragment order
  sp += (size_t)p.hidden * 2;
  // what the non-supplying lanes of an INT4 mma read: 256 bytes, entered 64 bytes in so that they fall on the other
  // half of the banks than the fragment words the supplying lanes read in the same 8-lane phase
  uint4 *zero = reinterpret_cast<uint4 *>(sp);
  sp += 384;
  float *xsum = reinterpret_cast<float *>(sp);  // per scale group: the sum of x, or (factor, offset) of the integer form
  sp += (size_t)(p.hidden / 32) * kMetaBytes;
  unsigned char *ring_ptr = sp + (size_t)warp * kWarpRingBytes;  // this warp's weight ring, then its scale stage
  sp += (size_t)kFusedWarps * kWarpRingBytes;
  const size_t wstage_bytes = (size_t)p.inter * 2 + (size_t)(p.inter / 32) * kMetaBytes;
  unsigned char *wstage = sp + (size_t)warp * wstage_bytes;  // this warp's private segment of mid
  sp += (size_t)kFusedWarps * wstage_bytes;
  int *w_ids = reinterpret_cast<int *>(sp);  // the CTA's copy of the routing
  sp += (size_t)kFusedWarps * 16 * 4;
  float *w_wts = reinterpret_cast<float *>(sp);
  sp += (size_t)kFusedWarps * 16 * 4;
  __shared__ int s_route_state;  // 0 nobody has it, 1 one warp is computing it, 2 ready
  if (tid == 0) s_route_state = 0;
  float *s_score = reinterpret_cast<float *>(sp);  // top-k scratch (one warp of the grid uses it)
  float *s_sel = s_score + p.experts;
  const uint32_t ring = (uint32_t)__cvta_generic_to_shared(ring_ptr);

  if (tid == 0) trace_cta(p, 0);
  for (int u = tid; u < p.hidden / 8; u += kFusedThreads) xnat[u] = reinterpret_cast<const uint4 *>(p.x)[u];
  {
    I4Stage st;
    st.xfrag = xfrag;
    st.zero = zero;
    st.xsum = xsum;
    stage_x_i4<false>(reinterpret_cast<const uint4 *>(p.x), st, p.hidden, 1, tid, kFusedThreads);
  }
  __syncthreads();
  if (tid == 0) trace_cta(p, 1);

  const bool supply = (t == (g & 3));
  XFragLane xl_x;  // fragments of x
  xl_x.ptr = supply ? xfrag + t : zero + 4 + t;
  xl_x.kb_stride = supply ? 16 : 0;
  XFragLane xl_m;  // fragments of this warp's staged mid
  xl_m.ptr = supply ? reinterpret_cast<const uint4 *>(wstage) + t : zero + 4 + t;
  xl_m.kb_stride = supply ? 16 : 0;
  float *msum = reinterpret_cast<float *>(wstage + (size_t)p.inter * 2);

  const unsigned epoch = p.ctrl[CTRL_EPOCH] + 1u;  // stable during the launch; the last CTA to leave bumps it
  unsigned *const err = p.ctrl + CTRL_ERROR;
  bool have_routing = false;

  // Queue index -> chunk.  B and C1 chunks need the routing (w_ids) to be in hand.
  auto decode = [&](unsigned c) {
    Chunk ch;
    if (c < p.cA0) {
      ch.kind = KIND_R;
      ch.rb = (int)c / p.cprR;
      ch.kc = (int)c - ch.rb * p.cprR;
      ch.k0 = ch.kc * p.spcR;
      ch.n = min(p.spcR, p.sprR - ch.k0);
      ch.slot = 0;
      const size_t wrow = p.hidden / 8;
      ch.w_lo = reinterpret_cast<const uint4 *>(p.router_w) + (size_t)(ch.rb * 16 + g) * wrow;
      ch.w_hi = ch.w_lo + 8 * wrow;
      ch.s_lo = ch.s_hi = nullptr;
      ch.s_stride = 0;
    } else if (c < p.cB0) {
      const int ci = (int)(c - p.cA0);
      ch.kind = KIND_A;
      ch.rb = ci / p.cprA;
      ch.kc = ci - ch.rb * p.cprA;
      ch.k0 = ch.kc * p.spcA;
      ch.n = min(p.spcA, p.sprA - ch.k0);
      ch.slot = p.topk;
      const size_t wrow = p.hidden / 8;
      ch.w_lo = reinterpret_cast<const uint4 *>(p.shared_gate) + (size_t)(ch.rb * 8 + g) * wrow;
      ch.w_hi = reinterpret_cast<const uint4 *>(p.shared_up) + (size_t)(ch.rb * 8 + g) * wrow;
      ch.s_lo = ch.s_hi = nullptr;
      ch.s_stride = 0;
    } else if (c < p.cC10) {
      const int ci = (int)(c - p.cB0);
      ch.kind = KIND_B;
      ch.rb = ci / p.cprB;
      ch.kc = ci - ch.rb * p.cprB;
      ch.k0 = ch.kc * p.spcB;
      ch.n = min(p.spcB, p.sprB - ch.k0);
      const int rb_per_slot = p.inter / 8;
      ch.slot = ch.rb / rb_per_slot;
      const int jb = ch.rb - ch.slot * rb_per_slot;
      const size_t wrow = p.hidden / 32;
      const size_t ebase0 = (size_t)w_ids[ch.slot] * p.inter * wrow + (size_t)(jb * 8) * wrow;
      const size_t ebase = ebase0 + (size_t)g * wrow;
      ch.w_lo = reinterpret_cast<const uint4 *>(p.gate_w) + ebase;
      ch.w_hi = reinterpret_cast<const uint4 *>(p.up_w) + ebase;
      ch.s_lo = p.gate_s + ebase0;
      ch.s_hi = p.up_s + ebase0;
      ch.s_stride = (int)wrow;
    } else if (c < p.cC20) {
      const int rb = (int)(c - p.cC10);
      const int rb_per_slot = p.hidden / 16;  // chunks per slot
      ch.kind = KIND_C1;
      ch.slot = rb / rb_per_slot;
      ch.rb = rb - ch.slot * rb_per_slot;  // output row-block
      ch.kc = 0;
      ch.k0 = 0;
      ch.n = p.sprC1;
      const size_t wrow = p.inter / 32;
      const size_t ebase = (size_t)w_ids[ch.slot] * p.hidden * wrow;
      ch.w_lo = reinterpret_cast<const uint4 *>(p.down_w) + ebase + (size_t)(ch.rb * 16 + g) * wrow;
      ch.w_hi = ch.w_lo + 8 * wrow;
      ch.s_lo = p.down_s + ebase + (size_t)(ch.rb * 16) * wrow;
      ch.s_hi = ch.s_lo + 8 * wrow;
      ch.s_stride = (int)wrow;
    } else {
      const int ci = (int)(c - p.cC20);
      ch.kind = KIND_C2;
      ch.rb = ci / p.cprC2;  // output row-block
      ch.kc = ci - ch.rb * p.cprC2;
      ch.k0 = ch.kc * p.spcC2;
      ch.n = min(p.spcC2, p.sprC2 - ch.k0);
      ch.slot = p.topk;
      const size_t wrow = p.shared_inter / 8;
      ch.w_lo = reinterpret_cast<const uint4 *>(p.shared_down) + (size_t)(ch.rb * 16 + g) * wrow;
      ch.w_hi = ch.w_lo + 8 * wrow;
      ch.s_lo = ch.s_hi = nullptr;
      ch.s_stride = 0;
    }
    return ch;
  };

  // The routing is computed once per CTA, by the first warp that needs it, from the tagged
  // logits (polled until the router's finishers have written them); same inputs, same rule,
  // so every CTA selects the same experts.  The other warps wait on a shared-memory flag.
  auto fetch_routing = [&]() {
    int st = 0;
    if (lane == 0) st = atomicCAS(&s_route_state, 0, 1);
    st = __shfl_sync(0xffffffffu, st, 0);
    if (st == 0) {
      for (int i0 = lane; i0 < p.experts; i0 += 32 * 4) {
        float lg[4];
        const int n = min(4, (p.experts - i0 + 31) / 32);
        ld_tagged_n<4>(p.logits + i0, 32, n, epoch, err, lg);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int i = i0 + 32 * j;
          if (j < n) {
            const float sc = 1.0f / (1.0f + expf(-lg[j]));
            s_score[i] = sc;
            s_sel[i] = sc + p.router_bias[i];
          }
        }
      }
      __syncwarp();
      int my_id;
      float my_w;
      warp_topk(s_score, s_sel, p.experts, p.topk, p.routed_scale, lane, my_id, my_w);
      if (lane < p.topk) {
        w_ids[lane] = my_id;
        w_wts[lane] = my_w;
        if (blockIdx.x == 0) {
          if (p.ids_out) p.ids_out[lane] = (uint16_t)my_id;
          if (p.wts_out) p.wts_out[lane] = my_w;
        }
      }
      __threadfence_block();
      __syncwarp();
      if (lane == 0) {
        atomicExch(&s_route_state, 2);
        if (blockIdx.x == 0) trace_launch(p, 1);
      }
    } else if (st == 1) {
      if (lane == 0) {
        unsigned it = 0;
        while (atomicAdd(&s_route_state, 0) != 2) {
          if (++it > kSpinLimit) {
            atomicExch(err, 1u);
            break;
          }
          __nanosleep(100);
        }
      }
      __syncwarp();
    }
    __threadfence_block();
    have_routing = true;
  };

  // Handing a finished chunk in: arrive() publishes the chunk's partial result as tagged
  // values and returns at once (no fence, no atomic).  The warp that holds the LAST chunk of
  // a row-block in queue order is its finisher: complete() makes it collect the other
  // chunks' values (polling a slot only if its writer is still at work), sum them in index
  // order and run the row-block's epilogue.  Chunks are handed out in order, so the chunks a
  // finisher waits for are already being worked on by warps that never wait for it.
  auto piece_part = [&](const Chunk &ch) { return ch.kind == KIND_R ? p.partR : ch.kind == KIND_A ? p.partA : ch.kind == KIND_B ? p.partB : p.partC2; };
  auto piece_n = [&](const Chunk &ch) { return ch.kind == KIND_R ? p.cprR : ch.kind == KIND_A ? p.cprA : ch.kind == KIND_B ? p.cprB : p.cprC2; };

  auto arrive = [&](const Chunk &ch, float v) {
    if (ch.kind == KIND_C1) {
      const float total = __shfl_sync(0xffffffffu, v, ((lane & 7) << 2) + ((lane >> 3) & 1) * 2);
      if (lane < 16) st_tagged(p.ys + (size_t)ch.slot * p.hidden + ch.rb * 16 + lane, round_bf16(total), epoch);
      return;
    }
    const int np = piece_n(ch);
    if (np > 1 && ch.kc != np - 1 && (t & 1) == 0)
      st_tagged(piece_part(ch) + ((size_t)ch.rb * np + ch.kc) * 16 + g + 8 * (t >> 1), v, epoch);
  };

  // out rows [ob*16, +16): every slot's contribution (tagged) weighted in slot order, plus the shared expert's
  auto combine_rows = [&](int ob, float own, int own_slot) {
    if (lane < 16) {
      float o = 0.f;
      for (int k0 = 0; k0 < p.topk; k0 += 4) {
        float yk[4];
        const int n = min(4, p.topk - k0);
        if (own_slot >= k0 && own_slot < k0 + n) {  // the own slot's value is not in memory: read the others one by one
#pragma unroll
          for (int j = 0; j < 4; ++j)
            yk[j] = (j >= n || k0 + j == own_slot) ? own : ld_tagged(p.ys + (size_t)(k0 + j) * p.hidden + ob * 16 + lane, epoch, err);
        } else {
          ld_tagged_n<4>(p.ys + (size_t)k0 * p.hidden + ob * 16 + lane, p.hidden, n, epoch, err, yk);
        }
#pragma unroll
        for (int j = 0; j < 4; ++j)
          if (j < n) o = fmaf(yk[j], w_wts[k0 + j], o);
      }
      o = round_bf16(o);
      if (p.shared_inter) o = round_bf16(o + own);
      p.y[ob * 16 + lane] = f32_to_bf16_bits(o);
    }
  };

  auto complete = [&](const Chunk &ch, float v) {
    if (ch.kind == KIND_C1) {
      // without a shared expert the last routed slot finishes the output rows
      if (p.shared_inter == 0 && ch.slot == p.topk - 1) {
        const float total = round_bf16(__shfl_sync(0xffffffffu, v, ((lane & 7) << 2) + ((lane >> 3) & 1) * 2));
        combine_rows(ch.rb, total, ch.slot);
      }
      return;
    }
    const int np = piece_n(ch);
    if (ch.kc != np - 1) return;
    float total = __shfl_sync(0xffffffffu, v, ((lane & 7) << 2) + ((lane >> 3) & 1) * 2);  // this chunk's rows in lanes 0..15
    if (np > 1 && lane < 16) {
      const uint2 *src = piece_part(ch) + (size_t)ch.rb * np * 16 + lane;
      float s = 0.f;
      for (int i0 = 0; i0 < np - 1; i0 += kCollect) {  // index order, then the own (last) chunk
        float part[kCollect];
        const int n = min(kCollect, np - 1 - i0);
        ld_tagged_n<kCollect>(src + (size_t)i0 * 16, 16, n, epoch, err, part);
#pragma unroll
        for (int j = 0; j < kCollect; ++j)
          if (j < n) s += part[j];
      }
      total = s + total;
    }
    if (ch.kind == KIND_R) {
      if (lane < 16) st_tagged(p.logits + ch.rb * 16 + lane, total, epoch);
      if (lane == 0) trace_launch(p, 5);
      return;
    }
    if (ch.kind == KIND_A || ch.kind == KIND_B) {
      const float up = __shfl_down_sync(0xffffffffu, total, 8);
      const int row0 = ch.kind == KIND_A ? ch.rb * 8 : (ch.rb - ch.slot * (p.inter / 8)) * 8;
      const uint32_t m = f32_to_bf16_bits(swiglu_ref_rounding(total, up));
      const uint32_t hi = __shfl_down_sync(0xffffffffu, m, 1);
      if (lane < 8 && (lane & 1) == 0)
        st_tagged(p.mid + ((size_t)ch.slot * p.mid_stride + row0 + lane) / 2, __uint_as_float(m | (hi << 16)), epoch);
      return;
    }
    // KIND_C2: the shared expert's rows are complete, and with them the output rows
    combine_rows(ch.rb, round_bf16(total), -1);
  };

  // The first chunk of every warp is its own index (no herd of atomics at the start); later
  // chunks come from the queue counter, fetched one chunk ahead.
  const unsigned W = gridDim.x * kFusedWarps;
  unsigned next = 0;
  unsigned c = blockIdx.x * kFusedWarps + warp;
  Chunk cur;
  cur.kind = KIND_NONE;
  if (c < p.total) {
    if (lane == 0) next = W + atomicAdd(p.ctrl + CTRL_QUEUE, 1u);
    if (c >= p.cB0 && c < p.cC20) fetch_routing();
    cur = decode(c);
    ring_prologue(cur, ring, lane);
  }
  int traced = 0;
  while (cur.kind != KIND_NONE) {
    // ---- the chunk's weights are in flight; now the activations -------------------------------
    float v;
    const bool tr = p.trace && warp == 1 && lane == 0 && traced < 2;
    if (tr) p.trace[16 + (size_t)blockIdx.x * kTraceSlots + 8 + traced * 4 + 0] = global_ns();
    if (cur.kind == KIND_C1 || cur.kind == KIND_C2) {
      if (!have_routing) fetch_routing();  // the combine needs the routing weights
      if (cur.kind == KIND_C1) {
        warp_stage_i4(p.mid + (size_t)cur.slot * p.mid_stride / 2, reinterpret_cast<uint4 *>(wstage), msum, p.inter, lane,
                      epoch, err);
        v = ring_consume(cur, ring, ring_ptr, xl_m, msum, nullptr, 0, lane);
      } else {
        uint4 *seg = reinterpret_cast<uint4 *>(wstage);
        const uint2 *src = p.mid + (size_t)p.topk * p.mid_stride / 2 + (size_t)cur.k0 * 16;
        for (int u0 = lane; u0 < cur.n * 4; u0 += 64) {
          uint4 vv[2];
          const int n = min(2, (cur.n * 4 - u0 + 31) / 32);
          ld_tagged_units<2>(src + (size_t)u0 * 4, 32 * 4, n, epoch, err, vv);
#pragma unroll
          for (int j = 0; j < 2; ++j)
            if (u0 + 32 * j < cur.n * 4) seg[u0 + 32 * j] = vv[j];
        }
        __syncwarp();
        v = ring_consume(cur, ring, ring_ptr, xl_m, msum, seg + t, cur.k0, lane);
      }
      __syncwarp();  // the staged segment is free again
    } else if (cur.kind == KIND_B) {
      v = ring_consume(cur, ring, ring_ptr, xl_x, xsum, nullptr, 0, lane);
    } else {
      v = ring_consume(cur, ring, ring_ptr, xl_x, xsum, xnat + t, 0, lane);
    }
    // ---- hand in (without waiting), put the next chunk's weights in flight, then look at the count ----
    if (tr) p.trace[16 + (size_t)blockIdx.x * kTraceSlots + 8 + traced * 4 + 1] = global_ns();
    arrive(cur, v);
    c = __shfl_sync(0xffffffffu, next, 0);
    Chunk nx;
    nx.kind = KIND_NONE;
    bool completed = false;
    if (c < p.total) {
      if (lane == 0) next = W + atomicAdd(p.ctrl + CTRL_QUEUE, 1u);
      if (c >= p.cB0 && c < p.cC20 && !have_routing) {
        // the routing may depend on the chunk in hand: finish it before waiting
        complete(cur, v);
        completed = true;
        fetch_routing();
      }
      nx = decode(c);
      ring_prologue(nx, ring, lane);
    }
    if (tr) p.trace[16 + (size_t)blockIdx.x * kTraceSlots + 8 + traced * 4 + 2] = global_ns();
    if (!completed) complete(cur, v);
    if (tr) p.trace[16 + (size_t)blockIdx.x * kTraceSlots + 8 + traced * 4 + 3] = global_ns(), ++traced;
    cur = nx;
  }

  if (blockIdx.x == 0 && warp == 0 && !have_routing) fetch_routing();  // CTA 0 reports the routing to the caller
  // ---- the last CTA to leave resets the launch-wide counters ------------------------------------
  cp_async_wait<0>();
  if (warp == 0 && lane == 0) trace_cta(p, 6);
  __syncthreads();
  if (tid == 0) {
    trace_cta(p, 7);
    const unsigned epoch_now = p.ctrl[CTRL_EPOCH] + 1u;
    __threadfence();
    unsigned old = atomicAdd(p.ctrl + CTRL_EXIT, 1u);
    if (old == gridDim.x - 1) {
      p.ctrl[CTRL_QUEUE] = 0;
      p.ctrl[CTRL_EXIT] = 0;
      p.ctrl[CTRL_EPOCH] = epoch_now;
      __threadfence();
      trace_launch(p, 3);
    }
  }
}

// ---------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------
static int ceil_div(int a, int b) { return (a + b - 1) / b; }

size_t fused_smem_bytes(const blok_moe_weights &w) {
  return (size_t)w.hidden * 4 + 384 + (size_t)(w.hidden / 32) * kMetaBytes + (size_t)kFusedWarps * kWarpRingBytes +
         (size_t)kFusedWarps * ((size_t)w.inter * 2 + (size_t)(w.inter / 32) * kMetaBytes) + (size_t)kFusedWarps * 16 * 8 +
         (size_t)w.experts * 2 * sizeof(float);
}

// Cuts a row-block of `spr` steps into equal chunks of about `target` steps.
static void cut(int spr, int target, int *spc, int *cpr) {
  *cpr = std::max(1, ceil_div(spr, target));
  *spc = std::max(1, ceil_div(spr, *cpr));
  *cpr = std::max(1, ceil_div(spr, *spc));
}

// Decides whether the fused kernel can serve this layer on the current device and,
// if so, fixes its chunking and sizes its scratch.  Returns BLOK_OK with
// plan->enabled set either way; a CUDA failure is an error.
int fused_plan(const blok_moe_weights &w, FusedPlan *plan) {
  plan->enabled = false;
  if (w.experts % 16 || w.topk > 16 || w.shared_inter % 32 || w.inter % 256 || w.hidden % 256) return BLOK_OK;
  if (w.experts_local != w.experts || w.expert_base != 0) return BLOK_OK;
  if (w.shared_inter > w.inter && w.shared_inter > 0 && 16 * 64 > w.inter * 2) return BLOK_OK;
  int dev = 0, coop = 0, sms = 0;
  BLOK_CUDA(cudaGetDevice(&dev));
  BLOK_CUDA(cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, dev));
  BLOK_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  if (!coop) return BLOK_OK;
  size_t smem = fused_smem_bytes(w);
  if (smem > 227 * 1024) return BLOK_OK;
  BLOK_CUDA(cudaFuncSetAttribute(moe_decode_fused_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  int per_sm = 0;
  BLOK_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, moe_decode_fused_kernel, kFusedThreads, smem));
  if (per_sm < 1) return BLOK_OK;
  plan->grid = sms;
  plan->smem = smem;
  plan->total_warps = plan->grid * kFusedWarps;
  // chunking (steps of 1 KB of weights per warp); BLOK_FUSED_CHUNK_STEPS="R,A,B,C2" overrides the target steps per
  // chunk of the four phases that are cut (a tuning aid; the defaults are the measured configuration)
  int tgt[4] = {14, 28, 14, 16};
  if (const char *e = getenv("BLOK_FUSED_CHUNK_STEPS")) {
    int v[4];
    if (sscanf(e, "%d,%d,%d,%d", &v[0], &v[1], &v[2], &v[3]) == 4 && v[0] > 0 && v[1] > 0 && v[2] > 0 && v[3] > 0)
      for (int i = 0; i < 4; ++i) tgt[i] = v[i];
  }
  plan->sprR = w.hidden / 32;
  cut(plan->sprR, tgt[0], &plan->spcR, &plan->cprR);
  plan->sprA = w.hidden / 32;
  cut(plan->sprA, tgt[1], &plan->spcA, &plan->cprA);
  plan->sprB = w.hidden / 128;
  cut(plan->sprB, tgt[2], &plan->spcB, &plan->cprB);
  plan->sprC1 = w.inter / 128;
  if (plan->spcB > kScaleMaxSteps || plan->sprC1 > kScaleMaxSteps) return BLOK_OK;  // an INT4 chunk's scales are staged whole
  plan->sprC2 = w.shared_inter / 32;
  plan->spcC2 = 1;
  plan->cprC2 = 1;
  if (w.shared_inter) cut(plan->sprC2, tgt[3], &plan->spcC2, &plan->cprC2);
  plan->nrbR = w.experts / 16;
  plan->nrbA = w.shared_inter / 8;
  plan->nrbB = w.topk * (w.inter / 8);
  plan->nrbC1 = w.topk * (w.hidden / 16);
  plan->nrbC2 = w.shared_inter ? w.hidden / 16 : 0;
  // a C2 chunk's activation segment must fit the per-warp staging area
  if ((size_t)plan->spcC2 * 64 > (size_t)w.inter * 2) return BLOK_OK;
  plan->enabled = true;
  return BLOK_OK;
}

int launch_moe_decode_fused(blok_moe_layer *L, const uint16_t *x, uint16_t *y, uint16_t *ids_out, float *wts_out,
                            cudaStream_t stream) {
  const blok_moe_weights &w = L->w;
  const FusedPlan &pl = L->plan;
  FusedParams p;
  p.hidden = w.hidden; p.inter = w.inter; p.experts = w.experts; p.topk = w.topk; p.shared_inter = w.shared_inter;
  p.routed_scale = w.routed_scale;
  p.router_w = w.router_w; p.router_bias = w.router_bias;
  p.gate_w = w.gate_w; p.up_w = w.up_w; p.down_w = w.down_w;
  p.gate_s = w.gate_s; p.up_s = w.up_s; p.down_s = w.down_s;
  p.shared_gate = w.shared_gate; p.shared_up = w.shared_up; p.shared_down = w.shared_down;
  p.x = x; p.y = y;
  p.ids_out = ids_out ? ids_out : L->ids;
  p.wts_out = wts_out ? wts_out : L->wts;
  p.logits = reinterpret_cast<uint2 *>(L->f_logits_t);
  p.mid = reinterpret_cast<uint2 *>(L->f_mid); p.mid_stride = L->f_mid_stride;
  p.ys = reinterpret_cast<uint2 *>(L->f_ys);
  p.partR = reinterpret_cast<uint2 *>(L->f_partR); p.partA = reinterpret_cast<uint2 *>(L->f_partA);
  p.partB = reinterpret_cast<uint2 *>(L->f_partB); p.partC2 = reinterpret_cast<uint2 *>(L->f_partC2);
  p.sprR = pl.sprR; p.spcR = pl.spcR; p.cprR = pl.cprR;
  p.sprA = pl.sprA; p.spcA = pl.spcA; p.cprA = pl.cprA;
  p.sprB = pl.sprB; p.spcB = pl.spcB; p.cprB = pl.cprB;
  p.sprC1 = pl.sprC1;
  p.sprC2 = pl.sprC2; p.spcC2 = pl.spcC2; p.cprC2 = pl.cprC2;
  p.cA0 = (unsigned)pl.nrbR * pl.cprR;
  p.cB0 = p.cA0 + (unsigned)pl.nrbA * pl.cprA;
  p.cC10 = p.cB0 + (unsigned)pl.nrbB * pl.cprB;
  p.cC20 = p.cC10 + (unsigned)pl.nrbC1;
  p.total = p.cC20 + (unsigned)pl.nrbC2 * pl.cprC2;
  p.ctrl = L->f_ctrl;
  p.trace = L->f_trace;
  void *args[] = {&p};
  BLOK_CUDA(cudaLaunchCooperativeKernel((const void *)moe_decode_fused_kernel, dim3(pl.grid), dim3(kFusedThreads), args,
                                        pl.smem, stream));
  return launch_status("moe_decode_fused_kernel");
}

}  // namespace blok
