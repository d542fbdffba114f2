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
//   R   router logits, bf16               16 rows x 8 k-steps per chunk
//   A   shared-expert gate/up, bf16       (8 gate + 8 up rows) x 16 k-steps
//   B   the selected experts' INT4 gate/up (8 + 8 rows) x 8 k-blocks; needs the routing
//   C1  INT4 down, one (slot, 16 output rows) block per chunk; needs every mid value
//   C2  shared-expert down, bf16          16 rows x 16 k-steps; needs the shared mid
//
// A chunk covers a row-block only partly.  Its 16 partial dot products go to a
// scratch slot indexed by the chunk's position in the row-block, and the warp that
// hands in the last chunk of a row-block (an arrival counter tells) sums the slots
// in index order and runs the row-block's epilogue: logits (and, for the last
// router row-block, the top-k for the whole grid), SiLU*up -> mid, or the
// per-slot down output whose 9th arrival triggers the weighted combine
//   y = bf16(bf16(sum_k w_k * bf16(y_k)) + bf16(shared)).
// Which warp computes a chunk varies from run to run; what is summed in which
// order does not, so results are deterministic.
//
// A warp that pulls a C chunk puts its weight loads in flight BEFORE it waits for
// the mid values, so the one real dependency of the layer costs little.  Every
// wait on another warp is a bounded spin that records an error word and goes on:
// the kernel always terminates.  The launch is cooperative (all CTAs resident).
#include <algorithm>
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
#define BLOK_RING_DEPTH 6
#endif
constexpr int kFusedWarps = BLOK_FUSED_WARPS;
constexpr int kFusedThreads = kFusedWarps * 32;
constexpr unsigned kSpinLimit = 1u << 22;  // polls before a wait gives up with an error word

enum { CTRL_QUEUE = 0, CTRL_ROUTER = 1, CTRL_ROUTED = 2, CTRL_MID = 3, CTRL_EXIT = 4, CTRL_ERROR = 5 };
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
  float *logits;   // [experts]
  int *route_ids;  // [topk] selected experts, published by the warp that runs the top-k
  float *route_wts;
  uint16_t *mid;   // [topk + 1][mid_stride] bf16; row topk is the shared expert's
  int mid_stride;
  float *ys;       // [topk + 1][hidden] bf16-valued per-slot down outputs
  float *partR, *partA, *partB, *partC2;
  unsigned *cntR, *cntA, *cntB, *cntC2, *cntOut;
  // chunking: steps per row-block, steps per chunk, chunks per row-block
  int sprR, spcR, cprR;
  int sprA, spcA, cprA;
  int sprB, spcB, cprB;
  int sprC1;
  int sprC2, spcC2, cprC2;
  unsigned cA0, cB0, cC10, cC20, total;  // first queue index of each phase; queue length
  unsigned mid_target;                    // row-blocks of A and B together
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

__device__ __forceinline__ unsigned ld_acquire_u32(const unsigned *p) {
  unsigned v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ unsigned atom_add_acq_rel(unsigned *p, unsigned v) {
  unsigned old;
  asm volatile("atom.acq_rel.gpu.global.add.u32 %0, [%1], %2;" : "=r"(old) : "l"(p), "r"(v) : "memory");
  return old;
}

// Lane 0 polls until *p >= target (bounded); the warp leaves together.
__device__ __forceinline__ void warp_wait(const unsigned *p, unsigned target, unsigned *err, unsigned code, int lane) {
  if (lane == 0) {
    unsigned it = 0;
    while (ld_acquire_u32(p) < target) {
      if (++it > kSpinLimit) {
        atomicExch(err, code);
        break;
      }
      __nanosleep(40);
    }
  }
  __syncwarp();
}

// The warp's earlier global writes become visible before lane 0's increment; the
// increment also acquires, so a warp that sees the final count may read what the
// other arrivals wrote.  Returns the old count in every lane.
__device__ __forceinline__ unsigned warp_arrive(unsigned *counter, int lane) {
  __syncwarp();
  unsigned old = 0;
  if (lane == 0) old = atom_add_acq_rel(counter, 1u);
  old = __shfl_sync(0xffffffffu, old, 0);
  return old;
}

// A warp hands in chunk `kc` of row-block `rb` (npieces chunks per row-block).  `v`
// is the chunk's partial dot product for A row g + 8*(t>>1) (lanes with even t).
// Returns true in the warp that completes the row-block, with the 16 row totals in
// lanes 0..15 (chunks summed in index order).
__device__ __forceinline__ bool hand_in_piece(float v, float *part, unsigned *cnt, int rb, int kc, int npieces,
                                              int lane, float &total) {
  const int g = lane >> 2, t = lane & 3;
  if (npieces == 1) {
    total = __shfl_sync(0xffffffffu, v, ((lane & 7) << 2) + ((lane >> 3) & 1) * 2);
    return true;
  }
  if ((t & 1) == 0) __stcg(part + ((size_t)rb * npieces + kc) * 16 + g + 8 * (t >> 1), v);
  const unsigned old = warp_arrive(cnt + rb, lane);
  if (old != (unsigned)(npieces - 1)) return false;
  float s = 0.f;
  if (lane < 16) {
    const float *src = part + (size_t)rb * npieces * 16 + lane;
    int i = 0;
    for (; i + 8 <= npieces; i += 8) {  // eight loads in flight, summed in index order
      float a[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) a[j] = __ldcg(src + (i + j) * 16);
#pragma unroll
      for (int j = 0; j < 8; ++j) s += a[j];
    }
    for (; i < npieces; ++i) s += __ldcg(src + i * 16);
  }
  total = s;
  if (lane == 0) cnt[rb] = 0;  // leave the counter clean for the next launch
  return true;
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
constexpr int kRingDepth = BLOK_RING_DEPTH;
constexpr int kRingStepBytes = 2 * 512 + 128;  // low rows, high rows, scales

__device__ __forceinline__ void cp_async16(uint32_t dst, const void *src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async4(uint32_t dst, const void *src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst), "l"(src) : "memory");
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
  const uint16_t *s_sel;     // the scale row this lane post-scales (INT4 kinds)
};

__device__ __forceinline__ bool kind_is_i4(int kind) { return kind == KIND_B || kind == KIND_C1; }

__device__ __forceinline__ void ring_issue(const Chunk &ch, int s, uint32_t ring, int lane) {
  if (s < ch.n) {
    const int t = lane & 3;
    const uint32_t base = ring + (uint32_t)(s % kRingDepth) * kRingStepBytes + (uint32_t)lane * 16;
    cp_async16(base, ch.w_lo + (size_t)(ch.k0 + s) * 4 + t);
    cp_async16(base + 512, ch.w_hi + (size_t)(ch.k0 + s) * 4 + t);
    if (kind_is_i4(ch.kind))
      cp_async4(ring + (uint32_t)(s % kRingDepth) * kRingStepBytes + 1024 + (uint32_t)lane * 4,
                ch.s_sel + (size_t)(ch.k0 + s) * 4);
  }
  cp_async_commit();
}

__device__ __forceinline__ void ring_prologue(const Chunk &ch, uint32_t ring, int lane) {
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
  for (int s = 0; s < ch.n; ++s) {
    cp_async_wait<kRingDepth - 1>();
    const unsigned char *slotp = ring_ptr + (size_t)(s % kRingDepth) * kRingStepBytes;
    const uint4 wl = *reinterpret_cast<const uint4 *>(slotp + lane * 16);
    const uint4 wh = *reinterpret_cast<const uint4 *>(slotp + 512 + lane * 16);
    const int kx = ch.k0 - kx0 + s;
    if (i4) {
      const uint32_t sc = *reinterpret_cast<const uint32_t *>(slotp + 1024 + lane * 4);
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

// One warp stages `cols` activation values (bf16, written earlier in this kernel by
// other CTAs, hence read through L2) into INT4 fragment order with group sums.
__device__ __forceinline__ void warp_stage_i4(const uint4 *src, uint4 *xfrag, float *xsum, int cols, int lane) {
  for (int u = lane; u < cols / 8; u += 32) {
    uint4 v = __ldcg(src + u);
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
  uint4 *zero = reinterpret_cast<uint4 *>(sp);  // what the non-supplying lanes of an INT4 mma read
  sp += 256;
  float *xsum = reinterpret_cast<float *>(sp);
  sp += (size_t)(p.hidden / 32) * 4;
  unsigned char *ring_ptr = sp + (size_t)warp * kRingDepth * kRingStepBytes;  // this warp's weight ring
  sp += (size_t)kFusedWarps * kRingDepth * kRingStepBytes;
  const size_t wstage_bytes = (size_t)p.inter * 2 + (size_t)(p.inter / 32) * 4;
  unsigned char *wstage = sp + (size_t)warp * wstage_bytes;  // this warp's private segment of mid
  sp += (size_t)kFusedWarps * wstage_bytes;
  int *w_ids = reinterpret_cast<int *>(sp) + warp * 16;  // this warp's copy of the routing
  sp += (size_t)kFusedWarps * 16 * 4;
  float *w_wts = reinterpret_cast<float *>(sp) + warp * 16;
  sp += (size_t)kFusedWarps * 16 * 4;
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
  xl_x.ptr = (supply ? xfrag : zero) + t;
  xl_x.kb_stride = supply ? 16 : 0;
  XFragLane xl_m;  // fragments of this warp's staged mid
  xl_m.ptr = (supply ? reinterpret_cast<const uint4 *>(wstage) : zero) + t;
  xl_m.kb_stride = supply ? 16 : 0;
  float *msum = reinterpret_cast<float *>(wstage + (size_t)p.inter * 2);

  bool have_routing = false;
  bool mid_ready = false;
  const int nrb_router = p.experts / 16;
  const unsigned ncontrib = (unsigned)p.topk + (p.shared_inter ? 1u : 0u);

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
      ch.s_sel = nullptr;
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
      ch.s_sel = nullptr;
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
      const size_t ebase = (size_t)w_ids[ch.slot] * p.inter * wrow + (size_t)(jb * 8 + g) * wrow;
      ch.w_lo = reinterpret_cast<const uint4 *>(p.gate_w) + ebase;
      ch.w_hi = reinterpret_cast<const uint4 *>(p.up_w) + ebase;
      ch.s_sel = ((t >> 1) ? p.up_s : p.gate_s) + ebase + 2 * (t & 1);
    } else if (c < p.cC20) {
      const int rb = (int)(c - p.cC10);
      const int rb_per_slot = p.hidden / 16;
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
      ch.s_sel = p.down_s + ebase + (size_t)(ch.rb * 16 + g + 8 * (t >> 1)) * wrow + 2 * (t & 1);
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
      ch.s_sel = nullptr;
    }
    return ch;
  };

  auto fetch_routing = [&]() {
    warp_wait(p.ctrl + CTRL_ROUTED, 1u, p.ctrl + CTRL_ERROR, 1u, lane);
    if (lane < p.topk) {
      w_ids[lane] = __ldcg(p.route_ids + lane);
      w_wts[lane] = __ldcg(p.route_wts + lane);
    }
    __syncwarp();
    have_routing = true;
  };

  // Hand the finished chunk in and run whatever epilogue its completion triggers.
  auto finish = [&](const Chunk &ch, float v) {
    float total;
    if (ch.kind == KIND_R) {
      if (!hand_in_piece(v, p.partR, p.cntR, ch.rb, ch.kc, p.cprR, lane, total)) return;
      if (lane < 16) __stcg(p.logits + ch.rb * 16 + lane, total);
      if (warp_arrive(p.ctrl + CTRL_ROUTER, lane) != (unsigned)nrb_router - 1) return;
      // every logit is in place: this warp selects the experts for the whole grid
      for (int i = lane; i < p.experts; i += 32) {
        float sc = 1.0f / (1.0f + expf(-__ldcg(p.logits + i)));
        s_score[i] = sc;
        s_sel[i] = sc + p.router_bias[i];
      }
      __syncwarp();
      int my_id;
      float my_w;
      warp_topk(s_score, s_sel, p.experts, p.topk, p.routed_scale, lane, my_id, my_w);
      if (lane < p.topk) {
        __stcg(p.route_ids + lane, my_id);
        __stcg(p.route_wts + lane, my_w);
        if (p.ids_out) p.ids_out[lane] = (uint16_t)my_id;
        if (p.wts_out) p.wts_out[lane] = my_w;
      }
      warp_arrive(p.ctrl + CTRL_ROUTED, lane);
      if (lane == 0) trace_launch(p, 1);
      return;
    }
    if (ch.kind == KIND_A || ch.kind == KIND_B) {
      const bool a = ch.kind == KIND_A;
      if (!hand_in_piece(v, a ? p.partA : p.partB, a ? p.cntA : p.cntB, ch.rb, ch.kc, a ? p.cprA : p.cprB, lane, total))
        return;
      const float up = __shfl_down_sync(0xffffffffu, total, 8);
      const int row0 = a ? ch.rb * 8 : (ch.rb - ch.slot * (p.inter / 8)) * 8;
      if (lane < 8) p.mid[(size_t)ch.slot * p.mid_stride + row0 + lane] = f32_to_bf16_bits(swiglu_ref_rounding(total, up));
      if (warp_arrive(p.ctrl + CTRL_MID, lane) == p.mid_target - 1 && lane == 0) trace_launch(p, 2);
      return;
    }
    if (ch.kind == KIND_C1) {
      total = __shfl_sync(0xffffffffu, v, ((lane & 7) << 2) + ((lane >> 3) & 1) * 2);
    } else {
      if (!hand_in_piece(v, p.partC2, p.cntC2, ch.rb, ch.kc, p.cprC2, lane, total)) return;
    }
    // this slot's contribution to output rows [rb*16, rb*16+16) is complete
    const int ob = ch.rb;
    if (lane < 16) __stcg(p.ys + (size_t)ch.slot * p.hidden + ob * 16 + lane, round_bf16(total));
    if (warp_arrive(p.cntOut + ob, lane) != ncontrib - 1) return;
    if (lane < 16) {
      float o = 0.f;
      for (int k = 0; k < p.topk; ++k) o = fmaf(__ldcg(p.ys + (size_t)k * p.hidden + ob * 16 + lane), w_wts[k], o);
      o = round_bf16(o);
      if (p.shared_inter) o = round_bf16(o + __ldcg(p.ys + (size_t)p.topk * p.hidden + ob * 16 + lane));
      p.y[ob * 16 + lane] = f32_to_bf16_bits(o);
    }
    if (lane == 0) p.cntOut[ob] = 0;
  };

  unsigned next = 0;
  if (lane == 0) next = atomicAdd(p.ctrl + CTRL_QUEUE, 1u);
  unsigned c = __shfl_sync(0xffffffffu, next, 0);
  Chunk cur;
  cur.kind = KIND_NONE;
  if (c < p.total) {
    if (lane == 0) next = atomicAdd(p.ctrl + CTRL_QUEUE, 1u);
    if (c >= p.cB0 && c < p.cC20) fetch_routing();
    cur = decode(c);
    ring_prologue(cur, ring, lane);
  }
  while (cur.kind != KIND_NONE) {
    // ---- the chunk's weights are in flight; now the activations -------------------------------
    float v;
    if (cur.kind == KIND_C1 || cur.kind == KIND_C2) {
      if (!have_routing) fetch_routing();  // the combine needs the routing weights
      if (!mid_ready) {
        warp_wait(p.ctrl + CTRL_MID, p.mid_target, p.ctrl + CTRL_ERROR, 2u, lane);
        mid_ready = true;
      }
      if (cur.kind == KIND_C1) {
        warp_stage_i4(reinterpret_cast<const uint4 *>(p.mid + (size_t)cur.slot * p.mid_stride),
                      reinterpret_cast<uint4 *>(wstage), msum, p.inter, lane);
        v = ring_consume(cur, ring, ring_ptr, xl_m, msum, nullptr, 0, lane);
      } else {
        uint4 *seg = reinterpret_cast<uint4 *>(wstage);
        const uint4 *src = reinterpret_cast<const uint4 *>(p.mid + (size_t)p.topk * p.mid_stride) + cur.k0 * 4;
        for (int u = lane; u < cur.n * 4; u += 32) seg[u] = __ldcg(src + u);
        __syncwarp();
        v = ring_consume(cur, ring, ring_ptr, xl_m, msum, seg + t, cur.k0, lane);
      }
      __syncwarp();  // the staged segment is free again
    } else if (cur.kind == KIND_B) {
      v = ring_consume(cur, ring, ring_ptr, xl_x, xsum, nullptr, 0, lane);
    } else {
      v = ring_consume(cur, ring, ring_ptr, xl_x, xsum, xnat + t, 0, lane);
    }
    // ---- next chunk: put its weights in flight before handing this one in -----------------------
    c = __shfl_sync(0xffffffffu, next, 0);
    Chunk nx;
    nx.kind = KIND_NONE;
    bool finished = false;
    if (c < p.total) {
      if (lane == 0) next = atomicAdd(p.ctrl + CTRL_QUEUE, 1u);
      if (c >= p.cB0 && c < p.cC20 && !have_routing) {
        // the routing may depend on the chunk in hand: hand it in before waiting
        finish(cur, v);
        finished = true;
        fetch_routing();
      }
      nx = decode(c);
      ring_prologue(nx, ring, lane);
    }
    if (!finished) finish(cur, v);
    cur = nx;
  }

  // ---- the last CTA to leave resets the launch-wide counters ------------------------------------
  cp_async_wait<0>();
  if (warp == 0 && lane == 0) trace_cta(p, 6);
  __syncthreads();
  if (tid == 0) {
    trace_cta(p, 7);
    __threadfence();
    unsigned old = atomicAdd(p.ctrl + CTRL_EXIT, 1u);
    if (old == gridDim.x - 1) {
      p.ctrl[CTRL_QUEUE] = 0;
      p.ctrl[CTRL_ROUTER] = 0;
      p.ctrl[CTRL_ROUTED] = 0;
      p.ctrl[CTRL_MID] = 0;
      p.ctrl[CTRL_EXIT] = 0;
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
  return (size_t)w.hidden * 4 + 256 + (size_t)(w.hidden / 32) * 4 + (size_t)kFusedWarps * kRingDepth * kRingStepBytes +
         (size_t)kFusedWarps * ((size_t)w.inter * 2 + (size_t)(w.inter / 32) * 4) + (size_t)kFusedWarps * 16 * 8 +
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
  // chunking (steps of 1 KB of weights per warp)
  plan->sprR = w.hidden / 32;
  cut(plan->sprR, 28, &plan->spcR, &plan->cprR);
  plan->sprA = w.hidden / 32;
  cut(plan->sprA, 28, &plan->spcA, &plan->cprA);
  plan->sprB = w.hidden / 128;
  cut(plan->sprB, 14, &plan->spcB, &plan->cprB);
  plan->sprC1 = w.inter / 128;
  plan->sprC2 = w.shared_inter / 32;
  plan->spcC2 = 1;
  plan->cprC2 = 1;
  if (w.shared_inter) cut(plan->sprC2, 32, &plan->spcC2, &plan->cprC2);
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
  p.logits = L->logits;
  p.route_ids = L->f_route_ids; p.route_wts = L->f_route_wts;
  p.mid = L->f_mid; p.mid_stride = L->f_mid_stride;
  p.ys = L->f_ys;
  p.partR = L->f_partR; p.partA = L->f_partA; p.partB = L->f_partB; p.partC2 = L->f_partC2;
  p.cntR = L->f_cntR; p.cntA = L->f_cntA; p.cntB = L->f_cntB; p.cntC2 = L->f_cntC2; p.cntOut = L->f_cntOut;
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
  p.mid_target = (unsigned)pl.nrbA + (unsigned)pl.nrbB;
  p.ctrl = L->f_ctrl;
  p.trace = L->f_trace;
  void *args[] = {&p};
  BLOK_CUDA(cudaLaunchCooperativeKernel((const void *)moe_decode_fused_kernel, dim3(pl.grid), dim3(kFusedThreads), args,
                                        pl.smem, stream));
  return launch_status("moe_decode_fused_kernel");
}

}  // namespace blok
