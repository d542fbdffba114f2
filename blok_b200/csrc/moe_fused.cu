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
//   R   router logits, bf16               16 rows x 14 k-steps per chunk
//   A   shared-expert gate/up, bf16       (8 gate + 8 up rows) x 28 k-steps
//   B   the selected experts' INT4 gate/up (8 + 8 rows) x 14 k-blocks; needs the routing
//   C1  INT4 down, one (slot, 16 output rows) block per chunk; needs that slot's mid values
//   C2  shared-expert down, bf16          16 rows x 32 k-steps; needs the shared mid
//
// Weights stream through a warp-private cp.async ring in shared memory (each lane copies and
// later reads back its own words, so the ring needs no barrier).  The INT4 chunks run on the
// integer tensor-core consumer of i4_imma.cuh (nibbles taken as bytes, activations as 15-bit
// block integers per scale group, exact int32 sums, scales applied per group in fp32): measured
// with this ring on a 148-CTA grid it sustains 6.0-6.4 TB/s where the bf16-operand consumer of
// i4_mma.cuh sustains 4.8-4.9 TB/s.
//
// A chunk covers a row-block only partly.  Its 16 partial dot products go to a
// scratch slot indexed by the chunk's position in the row-block, followed by one
// release/acquire increment of the row-block's counter.  The warp whose increment completes
// the row-block is its finisher (no warp ever waits for another chunk): it sums the slots in a
// fixed order and runs the row-block's epilogue: logits; SiLU*up -> mid; or, for the
// shared-expert down rows, the weighted combine of all nine contributions
//   y = bf16(bf16(sum_k w_k * bf16(y_k)) + bf16(shared)).
// Which warp computes a chunk varies from run to run; what is summed in which
// order does not, so results are deterministic.
//
// Hand-offs between warps:
//  - counters only grow (the value expected in launch n is n times the per-launch count, modulo 2^32), so
//    nothing is cleared between launches.
//  - the router's per-expert scores, the routing and the per-slot down outputs travel as 8-byte
//    (value, tag) pairs written with one store; the tag is the launch's epoch and a reader polls until
//    the tag matches.
//  - the mid vector of a slot (2,048 values, needed whole by every down chunk of the slot) is written
//    plainly, 16 bytes per row-block, followed by a fence and one increment of the slot's counter
//    (counters only grow: the value expected in launch n is n * row-blocks, modulo 2^32).  In every
//    CTA the first warp that needs a slot waits for its counter, quantises the vector ONCE into
//    shared memory for all 16 warps, and raises a shared-memory flag.
// The router's finishers publish, per expert, the selection value and the score as tagged pairs; one warp per CTA derives
// the routing from them when the CTA first needs it.  Every poll is bounded and records an
// error word read by blok_moe_layer_check; the launch is cooperative (all CTAs resident), so the warps
// being waited for are always running.
#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <vector>

#include "bf16_mma.cuh"
#include "i4_imma.cuh"
#include "moe_layer.h"
#include "router_topk.cuh"

namespace blok {

// 16 warps per CTA with 5 KB of weights in flight each: 20 warps and a ring of 6 steps measured the same (85-86 us),
// 8 warps and a ring of 4 slower.
constexpr int kFusedWarps = 16;
constexpr int kFusedThreads = kFusedWarps * 32;
constexpr unsigned kSpinLimit = 1u << 20;  // polls (about a microsecond apart once backed off) before a wait gives up with an error word
constexpr int kMaxTopk = 16;

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
  uint2 *logits;      // [2][experts] per expert (sel = sigmoid(logit) + bias, launch tag), then (sigmoid(logit), launch tag)
  int r_local;        // 1: the chunks of a router row-block are exactly one CTA's first chunks and are reduced in shared memory
  uint32_t *mid;      // [topk + 1][mid_stride / 2] bf16 pairs, plain; row topk is the shared expert's
  unsigned *mid_cnt;  // [topk + 1] row-blocks of mid written so far, over all launches
  int mid_stride;
  uint2 *ys;          // [topk][hidden] (bf16-valued per-slot down output, launch tag)
  float *partR, *partA, *partB, *partC2;  // [row-block][chunk][16] partial dot products of the chunks of a row-block
  unsigned *cntR, *cntA, *cntB, *cntC2;   // [row-block] chunks of the row-block handed in so far, over all launches
  // chunking: steps per row-block, steps per chunk, chunks per row-block
  int sprR, spcR, cprR;
  int sprA, spcA, cprA;
  int sprB, spcB, cprB;
  int sprC1;
  int sprC2, spcC2, cprC2;
  unsigned cA0, cB0, cC10, cC20, total;  // first queue index of each phase; queue length
  float inv_cprR, inv_cprA, inv_cprB, inv_cprC2, inv_rbB, inv_rbC1;  // reciprocals of the divisors of the queue-index arithmetic
  unsigned *ctrl;
  unsigned *err_host;  // optional: pinned host word that receives the launch's error word when the last CTA leaves
  // A rank's share of the layer (experts split over ranks): part_out != NULL.  The gate/up/down arrays then hold experts
  // [expert_base, expert_base + experts_local) only, the queue carries the B and C1 chunks of the selected experts that lie
  // in that range (the others' are another rank's work), and instead of y the kernel writes part_out[hidden] = the
  // weighted sum of those experts' outputs, fp32 and unrounded, and shared_out[hidden] = the shared expert's output.
  int expert_base, experts_local;
  float *part_out;
  uint16_t *shared_out;
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

// A waiting warp must not eat the issue slots of the warps it waits for (it shares a scheduler with three others): every
// poll loop sleeps between polls, longer each time, up to about a microsecond.
__device__ __forceinline__ void backoff(unsigned &ns) {
  __nanosleep(ns);
  ns = min(ns * 2u, 1024u);
}
// q = a / b for small non-negative a (< 2^22), with inv = 1 / b as a float: no integer division in the per-chunk code.
__device__ __forceinline__ int div_small(int a, float inv) { return (int)(((float)a + 0.5f) * inv); }

// ---- tagged hand-offs ---------------------------------------------------------------------------
__device__ __forceinline__ void st_tagged(uint2 *p, float v, unsigned tag) {
  asm volatile("st.global.cg.v2.u32 [%0], {%1, %2};" ::"l"(p), "r"(__float_as_uint(v)), "r"(tag) : "memory");
}
// N tagged values at p[0], p[stride], ...: all loads are issued before any tag is looked at,
// so the wait is one memory round trip, not N; the batch is re-read only while a tag is missing.
template <int N>
__device__ __forceinline__ void ld_tagged_n(const uint2 *p, int stride, int n, unsigned tag, unsigned *err, float (&out)[N]) {
  unsigned v[N], tg[N];
  unsigned ns = 32;
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
    backoff(ns);
  }
#pragma unroll
  for (int i = 0; i < N; ++i) out[i] = i < n ? __uint_as_float(v[i]) : 0.f;
}

// Hands a chunk's results in: one release + acquire increment of the row-block's counter (the partial sums stored by the
// warp's lanes before the __syncwarp are covered by it).  Returns the counter's value before the increment.
__device__ __forceinline__ unsigned arrive_counter(unsigned *cnt) {
  unsigned old;
  asm volatile("atom.add.acq_rel.gpu.global.u32 %0, [%1], 1;" : "=r"(old) : "l"(cnt) : "memory");
  return old;
}

__device__ __forceinline__ unsigned ld_acquire_gpu(const unsigned *p) {
  unsigned v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
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
constexpr int kRingDepth = 5;
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

// w_lo / w_hi: the lane's two weight rows at the chunk's first step (+ t), n: steps of the chunk
__device__ __forceinline__ void ring_issue(const uint4 *w_lo, const uint4 *w_hi, int n, int s, uint32_t ring, int lane) {
  if (s < n) {
    const uint32_t base = ring + (uint32_t)(s % kRingDepth) * kRingStepBytes + (uint32_t)lane * 16;
    cp_async16(base, w_lo + (size_t)s * 4);
    cp_async16(base + 512, w_hi + (size_t)s * 4);
  }
  cp_async_commit();
}

// The chunk's scales, whole: 16 rows x n k-blocks x 8 bytes, into the warp's scale stage (behind the ring).
__device__ __forceinline__ void scale_issue(const Chunk &ch, uint32_t ring, int lane) {
  const uint32_t stage = ring + kRingDepth * kRingStepBytes;
  const int pieces = 16 * ch.n;
  const float inv_n = 1.0f / (float)ch.n;
  for (int pc = lane; pc < pieces; pc += 32) {
    const int row = div_small(pc, inv_n), s = pc - row * ch.n;
    const uint16_t *src = ((row & 8) ? ch.s_hi : ch.s_lo) + (size_t)(row & 7) * ch.s_stride + (size_t)(ch.k0 + s) * 4;
    cp_async8(stage + (uint32_t)(row * kScaleRowBytes + s * 8), src);
  }
}

__device__ __forceinline__ void ring_prologue(const Chunk &ch, uint32_t ring, int lane) {
  __syncwarp();  // every lane is done with the previous chunk's scales
  if (kind_is_i4(ch.kind)) scale_issue(ch, ring, lane);  // joins the first step's commit group
  const uint4 *w_lo = ch.w_lo + (size_t)ch.k0 * 4 + (lane & 3), *w_hi = ch.w_hi + (size_t)ch.k0 * 4 + (lane & 3);
#pragma unroll
  for (int i = 0; i < kRingDepth; ++i) ring_issue(w_lo, w_hi, ch.n, i, ring, lane);
}

// The two streaming loops are kept out of line with plain arguments: they then get registers of their own, and what the
// chunk-level code around them keeps alive is saved once per chunk, not spilled inside the loops.
//
// bf16 weights: the chunk's partial dot product for A row g + 8 * (t >> 1).  w_lo / w_hi: the lane's weight rows at the
// chunk's first step (+ t); xrow: the activations of that step (bf16, natural order, + t).
// What a streaming loop hands back: the chunk's partial dot product and, in lane 0, the warp's next queue index.  The index
// is drawn when only a ring's worth of steps is left, not a whole chunk ahead: a chunk that has been handed out is then
// being worked on within one chunk's time, which is what every dependent (the routing, a slot's mid vector) waits for.
struct Consumed {
  float v;
  unsigned next;
};
__device__ __forceinline__ void draw_next(int s, int n, unsigned *queue, unsigned W, int lane, unsigned &next) {
  if (s == max(n - kRingDepth - 2, 0) && lane == 0) next = W + atomicAdd(queue, 1u);
}

__device__ __noinline__ Consumed consume_bf16(const uint4 *w_lo, const uint4 *w_hi, int n, uint32_t ring, const unsigned char *ring_ptr,
                                              const uint4 *xrow, unsigned *queue, unsigned W, int lane) {
  float d[4] = {0.f, 0.f, 0.f, 0.f};
  unsigned next = 0;
  for (int s = 0; s < n; ++s) {
    draw_next(s, n, queue, W, lane, next);
    cp_async_wait<kRingDepth - 1>();
    const unsigned char *slotp = ring_ptr + (size_t)(s % kRingDepth) * kRingStepBytes;
    const uint4 wl = *reinterpret_cast<const uint4 *>(slotp + lane * 16);
    const uint4 wh = *reinterpret_cast<const uint4 *>(slotp + 512 + lane * 16);
    const uint4 xb = xrow[s * 4];
    mma_bf16_16816(d, wl.x, wh.x, wl.y, wh.y, xb.x, xb.y);
    mma_bf16_16816(d, wl.z, wh.z, wl.w, wh.w, xb.z, xb.w);
    ring_issue(w_lo, w_hi, n, s + kRingDepth, ring, lane);
  }
  return Consumed{(lane & 2) ? d[2] : d[0], next};
}

// INT4 weights on the integer tensor-core consumer: activations staged by imma_stage_unit (bytes, per-group meta).
// xp: the lane's operand words of the chunk's first k-block (stride xstride uint4 per k-block); meta: that k-block's
// groups.  Every lane post-scales its own scale group (t) of rows g and g + 8; the quad is summed at the end.
// Returns the chunk's partial dot product: row g in lanes t < 2, row g + 8 in lanes t >= 2.
__device__ __noinline__ Consumed consume_i4(const uint4 *w_lo, const uint4 *w_hi, int n, uint32_t ring, const unsigned char *ring_ptr,
                                            const uint4 *xp, int xstride, const uint2 *meta, unsigned *queue, unsigned W, int lane) {
  const int g = lane >> 2, t = lane & 3;
  float acc_lo = 0.f, acc_hi = 0.f;
  unsigned next = 0;
  const unsigned char *sc_lo = ring_ptr + kRingDepth * kRingStepBytes + g * kScaleRowBytes + t * 2;
  const unsigned char *sc_hi = sc_lo + 8 * kScaleRowBytes;
  meta += t;
  // one k-block per turn; two per turn (independent unpack / MMA / post-scale streams) measured no faster
  for (int s = 0; s < n; ++s) {
    draw_next(s, n, queue, W, lane, next);
    cp_async_wait<kRingDepth - 1>();
    if (s == 0) __syncwarp();
    const unsigned char *slotp = ring_ptr + (size_t)(s % kRingDepth) * kRingStepBytes;
    const uint4 wl = *reinterpret_cast<const uint4 *>(slotp + lane * 16);
    const uint4 wh = *reinterpret_cast<const uint4 *>(slotp + 512 + lane * 16);
    const float s_lo = bf16_bits_to_f32(*reinterpret_cast<const uint16_t *>(sc_lo + s * 8));
    const float s_hi = bf16_bits_to_f32(*reinterpret_cast<const uint16_t *>(sc_hi + s * 8));
    int di[4] = {0, 0, 0, 0};
    imma_kblock(wl, wh, xp + s * xstride, di);
    imma_post(di, meta[s * 4], s_lo, s_hi, acc_lo, acc_hi);
    ring_issue(w_lo, w_hi, n, s + kRingDepth, ring, lane);
  }
  acc_lo += __shfl_xor_sync(0xffffffffu, acc_lo, 1);
  acc_lo += __shfl_xor_sync(0xffffffffu, acc_lo, 2);
  acc_hi += __shfl_xor_sync(0xffffffffu, acc_hi, 1);
  acc_hi += __shfl_xor_sync(0xffffffffu, acc_hi, 2);
  return Consumed{(t & 2) ? acc_hi : acc_lo, next};
}

// Shared-memory flag of something one warp of the CTA prepares for all: 0 nobody has it, 1 in progress, 2 ready.
// Returns true to exactly one warp (the one that has to prepare it); the others return false once it is ready.
__device__ __forceinline__ bool claim_or_wait(int *state, int lane, unsigned *err, unsigned code) {
  int st = 0;
  if (lane == 0) st = atomicCAS(state, 0, 1);
  st = __shfl_sync(0xffffffffu, st, 0);
  if (st == 0) return true;
  if (st == 1) {
    if (lane == 0) {
      unsigned it = 0, ns = 64;
      while (*reinterpret_cast<volatile int *>(state) != 2) {
        if (++it > kSpinLimit) {
          atomicExch(err, code);
          break;
        }
        backoff(ns);
      }
    }
    __syncwarp();
  }
  __threadfence_block();
  return false;
}
__device__ __forceinline__ void publish(int *state, int lane) {
  __threadfence_block();
  __syncwarp();
  if (lane == 0) atomicExch(state, 2);
}

// ---- the rare, register-hungry parts, kept out of line so that the streaming loops keep their registers ----------

// The routing (src/kimi_exec.cu:382-397): k rounds of argmax over sel = sigmoid(logit) + bias with strict '>' scanning
// ascending indices, so the lowest index wins a tie and NaN is never chosen; weights s / (sum + 1e-20) * routed_scale, the
// sum taken in selection order.  The router's finishers publish sel and s per expert as tagged values; one warp per CTA
// (the first that needs the routing) derives it from them: same inputs, same rule, so every CTA selects the same experts,
// and no CTA waits for another to publish a result.  Lane l keeps experts l, l + 32, ... in registers together with its
// own best; a round is one butterfly over the lanes' bests, and only the winning lane looks for its next best.
template <int NREG>  // candidates per lane: experts <= 32 * NREG
__device__ __noinline__ void routing_from_scores(const uint2 *sel_t, const uint2 *score_t, int *w_ids, float *w_wts, uint16_t *ids_out,
                                                 float *wts_out, int experts, int topk, float routed_scale, unsigned epoch, unsigned *err,
                                                 int lane) {
  float sel[NREG];
  {
    const int n = max(0, min(NREG, (experts - lane + 31) / 32));
    ld_tagged_n<NREG>(sel_t + lane, 32, n, epoch, err, sel);  // all of the lane's candidates in one round trip
#pragma unroll
    for (int j = 0; j < NREG; ++j)
      if (j >= n) sel[j] = -INFINITY;
  }
  float lb = -INFINITY;  // this lane's best candidate and its register
  int lj = -1;
#pragma unroll
  for (int j = 0; j < NREG; ++j)
    if (sel[j] > lb) lb = sel[j], lj = j;
  int my_id = 0;
  unsigned s_bits = 0, s_tag = epoch;
  for (int k = 0; k < topk; ++k) {
    float best = lb;
    int id = lj >= 0 ? lane + 32 * lj : 0x7fffffff;
#pragma unroll
    for (int o = 16; o; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, id, o);
      if (ob > best || (ob == best && oi < id)) best = ob, id = oi;
    }
    const bool mine = lj >= 0 && id == lane + 32 * lj;
    if (id == 0x7fffffff) id = 0;  // every candidate left is -inf or NaN: the reference keeps id 0
    if (lane == k) {  // the winner's score is requested now and looked at after the last round
      my_id = id;
      asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];" : "=r"(s_bits), "=r"(s_tag) : "l"(score_t + id) : "memory");
    }
    if (mine) {  // the chosen one leaves the pool; its lane finds its next best
      lb = -INFINITY;
      const int gone = lj;
      lj = -1;
#pragma unroll
      for (int j = 0; j < NREG; ++j) {
        if (j == gone) sel[j] = -INFINITY;
        if (sel[j] > lb) lb = sel[j], lj = j;
      }
    }
  }
  float my_s = __uint_as_float(s_bits);
  if (lane < topk && s_tag != epoch) {  // sel was there but its score's store had not landed yet: wait for it
    float v[1];
    ld_tagged_n<1>(score_t + my_id, 0, 1, epoch, err, v);
    my_s = v[0];
  }
  if (lane >= topk) my_s = 0.f;
  float sum = 0.f;
  for (int k = 0; k < topk; ++k) sum += __shfl_sync(0xffffffffu, my_s, k);  // selection order, as the reference adds
  const float my_w = my_s / (sum + 1.0e-20f) * routed_scale;
  if (lane < topk) {
    w_ids[lane] = my_id;
    w_wts[lane] = my_w;
    if (ids_out) ids_out[lane] = (uint16_t)my_id;
    if (wts_out) wts_out[lane] = my_w;
  }
}

// x -> shared memory: bf16 as it lies (operand of the bf16 chunks) and block integers (operand of the INT4 gate/up chunks).
// A thread's loads are all issued before anything is done with them: one memory round trip for the whole vector.
__device__ __noinline__ void stage_x_both(const uint16_t *x, uint4 *xnat, unsigned char *xq, uint2 *meta, uint4 *zero, int hidden, int tid) {
  const int units = hidden / 8;  // a multiple of 32: the four units of a scale group sit in four adjacent, live lanes
  const uint4 *src = reinterpret_cast<const uint4 *>(x);
  for (int u0 = 0; u0 < units; u0 += 2 * kFusedThreads) {
    const int ua = u0 + tid, ub = ua + kFusedThreads;
    const bool la = ua < units, lb = ub < units;
    const uint4 va = la ? src[ua] : make_uint4(0, 0, 0, 0);
    const uint4 vb = lb ? src[ub] : make_uint4(0, 0, 0, 0);
    if (la) xnat[ua] = va;
    if (lb) xnat[ub] = vb;
    imma_stage_unit(va, ua, la, xq, meta);
    imma_stage_unit(vb, ub, lb, xq, meta);
  }
  for (int u = tid; u < 8; u += kFusedThreads) zero[u] = make_uint4(0, 0, 0, 0);
}

// Waits until `row_blocks` more row-blocks of a slot's mid vector have been written in this launch.
__device__ __forceinline__ void wait_mid_counter(const unsigned *cnt, int row_blocks, unsigned epoch, unsigned *err, int lane) {
  if (lane == 0) {
    const unsigned want = epoch * (unsigned)row_blocks;  // counters only grow; modulo 2^32 like the epoch itself
    unsigned it = 0, ns = 64;
    while ((int)(ld_acquire_gpu(cnt) - want) < 0) {
      if (++it > kSpinLimit) {
        atomicExch(err, 2u);
        break;
      }
      backoff(ns);
    }
  }
  __syncwarp();
}

// A routed slot's mid vector -> block integers in shared memory (one warp, once per CTA and slot).
__device__ __noinline__ void stage_mid_i4(const unsigned *cnt, const uint32_t *mid_row, int inter, unsigned char *dst, unsigned epoch,
                                          unsigned *err, int lane) {
  wait_mid_counter(cnt, inter / 8, epoch, err, lane);
  const uint4 *src = reinterpret_cast<const uint4 *>(mid_row);
  uint2 *meta = reinterpret_cast<uint2 *>(dst + (size_t)inter * 2);
  const int units = inter / 8;  // a multiple of 32: a scale group's four units sit in four adjacent lanes
  for (int u = lane; u < units; u += 32) imma_stage_unit(__ldcg(src + u), u, true, dst, meta);
}

// The shared expert's mid vector, bf16 as it lies.
__device__ __noinline__ void stage_mid_bf16(const unsigned *cnt, const uint32_t *mid_row, int shared_inter, uint4 *smid, unsigned epoch,
                                            unsigned *err, int lane) {
  wait_mid_counter(cnt, shared_inter / 8, epoch, err, lane);
  const uint4 *src = reinterpret_cast<const uint4 *>(mid_row);
  for (int u = lane; u < shared_inter / 8; u += 32) smid[u] = __ldcg(src + u);
}

// out rows [ob*16, +16): every slot's contribution (tagged) weighted in slot order, plus the shared expert's
__device__ __noinline__ void combine_rows(const uint2 *ys, uint16_t *y, int hidden, int topk, bool has_shared, const float *w_wts, int ob,
                                          float shared_val, unsigned epoch, unsigned *err, int lane, float *part_out,
                                          uint16_t *shared_out) {
  if (lane < 16) {
    float o = 0.f;
    for (int k0 = 0; k0 < topk; k0 += 8) {
      float yk[8];
      const int n = min(8, topk - k0);
      ld_tagged_n<8>(ys + (size_t)k0 * hidden + ob * 16 + lane, hidden, n, epoch, err, yk);
#pragma unroll
      for (int j = 0; j < 8; ++j)
        if (j < n) o = fmaf(yk[j], w_wts[k0 + j], o);
    }
    if (part_out) {  // a rank's share: the other ranks' sums are added before anything is rounded
      part_out[ob * 16 + lane] = o;
      shared_out[ob * 16 + lane] = f32_to_bf16_bits(shared_val);
      return;
    }
    o = round_bf16(o);
    if (has_shared) o = round_bf16(o + shared_val);
    y[ob * 16 + lane] = f32_to_bf16_bits(o);
  }
}

// The warp that hands in the LAST chunk of a row-block (it learns so from the row-block's counter) is its finisher: every
// chunk's partial sums are in memory by then (each was followed by a release on the counter), and it adds them in chunk
// order: lane (half, row) takes chunks half, half + 2, ..., the two halves are added last.  Lanes 0..15 return the rows.
__device__ __noinline__ float collect_row_block(const float *part_rb, int np, int lane) {
  const int half = lane >> 4, row = lane & 15;
  const float *src = part_rb + row;
  float s = 0.f;
  for (int i0 = half; i0 < np; i0 += 32) {
    float pv[16];
#pragma unroll
    for (int j = 0; j < 16; ++j) pv[j] = i0 + 2 * j < np ? __ldcg(src + (size_t)(i0 + 2 * j) * 16) : 0.f;
#pragma unroll
    for (int j = 0; j < 16; ++j) s += pv[j];
  }
  return s + __shfl_down_sync(0xffffffffu, s, 16);
}

// Epilogue of a gate/up row-block: rows 0..7 gate, 8..15 up (lanes 0..15 of `total`) -> eight mid values = 16 bytes,
// written by one lane, then a fence and the slot's counter.  Returns the counter's value before the increment (lane 0).
__device__ __noinline__ unsigned publish_mid(float total, uint32_t *dst, unsigned *cnt, int lane) {
  const float up = __shfl_down_sync(0xffffffffu, total, 8);
  const uint32_t m = f32_to_bf16_bits(swiglu_ref_rounding(total, up));
  const uint32_t pair = m | (__shfl_down_sync(0xffffffffu, m, 1) << 16);  // lanes 0, 2, 4, 6 hold the pairs
  uint4 out;
  out.x = __shfl_sync(0xffffffffu, pair, 0);
  out.y = __shfl_sync(0xffffffffu, pair, 2);
  out.z = __shfl_sync(0xffffffffu, pair, 4);
  out.w = __shfl_sync(0xffffffffu, pair, 6);
  unsigned before = 0;
  if (lane == 0) {
    *reinterpret_cast<uint4 *>(dst) = out;
    __threadfence();
    before = atomicAdd(cnt, 1u);
  }
  return before;
}

__global__ void __launch_bounds__(kFusedThreads, 1) moe_decode_fused_kernel(const FusedParams p) {
  extern __shared__ __align__(16) unsigned char smem[];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t = lane & 3;

  // ---- shared memory carve-up -------------------------------------------------
  unsigned char *sp = smem;
  uint4 *xnat = reinterpret_cast<uint4 *>(sp);  // x, natural order (bf16 operand of R and A)
  sp += (size_t)p.hidden * 2;
  ImmaStage xq = imma_stage_carve(sp, p.hidden);  // x as block integers (operand of B); its zero region serves every INT4 chunk
  sp += imma_stage_bytes(p.hidden);
  const size_t midq_bytes = (size_t)p.inter * 2 + (size_t)(p.inter / 32) * 8;
  unsigned char *midq = sp;  // [topk] a slot's mid vector as block integers (operand of C1), staged once per CTA
  sp += (size_t)p.topk * midq_bytes;
  uint4 *smid = reinterpret_cast<uint4 *>(sp);  // the shared expert's mid, bf16 natural order (operand of C2)
  sp += (size_t)p.shared_inter * 2;
  unsigned char *ring_ptr = sp + (size_t)warp * kWarpRingBytes;  // this warp's weight ring, then its scale stage
  sp += (size_t)kFusedWarps * kWarpRingBytes;
  __shared__ int w_ids[kMaxTopk];    // the CTA's copy of the routing
  __shared__ float w_wts[kMaxTopk];
  __shared__ float s_rpart[kFusedWarps][16];  // router row-block reduced inside the CTA (r_local)
  __shared__ int s_rcount;
  __shared__ int s_route_state;
  __shared__ int s_mid_state[kMaxTopk + 1];  // [slot]; entry topk is the shared expert's mid
  __shared__ unsigned s_bound[3];  // first queue index of C1 and of C2, queue length: a rank's share shortens B and C1
  __shared__ int s_slots;          // routed slots in the queue: topk, or the selected experts this rank holds
  __shared__ int s_last;
  if (tid == 0) s_route_state = 0, s_rcount = 0, s_bound[0] = p.cC10, s_bound[1] = p.cC20, s_bound[2] = p.total, s_slots = p.topk;
  if (tid <= kMaxTopk) s_mid_state[tid] = 0;
  const uint32_t ring = (uint32_t)__cvta_generic_to_shared(ring_ptr);

  const unsigned epoch = p.ctrl[CTRL_EPOCH] + 1u;  // stable during the launch; the last CTA to leave bumps it
  unsigned *const err = p.ctrl + CTRL_ERROR;
  bool have_routing = false;
  if (tid == 0) trace_cta(p, 0);

  // Queue index -> chunk.  B and C1 chunks need the routing (w_ids) to be in hand.
  auto decode = [&](unsigned c) {
    Chunk ch;
    ch.s_lo = ch.s_hi = nullptr;
    ch.s_stride = 0;
    if (c < p.cA0) {
      ch.kind = KIND_R;
      ch.rb = div_small((int)c, p.inv_cprR);
      ch.kc = (int)c - ch.rb * p.cprR;
      ch.k0 = ch.kc * p.spcR;
      ch.n = min(p.spcR, p.sprR - ch.k0);
      ch.slot = 0;
      const size_t wrow = p.hidden / 8;
      ch.w_lo = reinterpret_cast<const uint4 *>(p.router_w) + (size_t)(ch.rb * 16 + g) * wrow;
      ch.w_hi = ch.w_lo + 8 * wrow;
    } else if (c < p.cB0) {
      const int ci = (int)(c - p.cA0);
      ch.kind = KIND_A;
      ch.rb = div_small(ci, p.inv_cprA);
      ch.kc = ci - ch.rb * p.cprA;
      ch.k0 = ch.kc * p.spcA;
      ch.n = min(p.spcA, p.sprA - ch.k0);
      ch.slot = p.topk;
      const size_t wrow = p.hidden / 8;
      ch.w_lo = reinterpret_cast<const uint4 *>(p.shared_gate) + (size_t)(ch.rb * 8 + g) * wrow;
      ch.w_hi = reinterpret_cast<const uint4 *>(p.shared_up) + (size_t)(ch.rb * 8 + g) * wrow;
    } else if (c < s_bound[0]) {
      const int ci = (int)(c - p.cB0);
      ch.kind = KIND_B;
      ch.rb = div_small(ci, p.inv_cprB);
      ch.kc = ci - ch.rb * p.cprB;
      ch.k0 = ch.kc * p.spcB;
      ch.n = min(p.spcB, p.sprB - ch.k0);
      const int rb_per_slot = p.inter / 8;
      ch.slot = div_small(ch.rb, p.inv_rbB);
      const int jb = ch.rb - ch.slot * rb_per_slot;
      const size_t wrow = p.hidden / 32;
      const size_t ebase0 = (size_t)w_ids[ch.slot] * p.inter * wrow + (size_t)(jb * 8) * wrow;
      const size_t ebase = ebase0 + (size_t)g * wrow;
      ch.w_lo = reinterpret_cast<const uint4 *>(p.gate_w) + ebase;
      ch.w_hi = reinterpret_cast<const uint4 *>(p.up_w) + ebase;
      ch.s_lo = p.gate_s + ebase0;
      ch.s_hi = p.up_s + ebase0;
      ch.s_stride = (int)wrow;
    } else if (c < s_bound[1]) {
      const int rb = (int)(c - s_bound[0]);
      const int rb_per_slot = p.hidden / 16;  // chunks per slot
      ch.kind = KIND_C1;
      ch.slot = div_small(rb, p.inv_rbC1);
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
      const int ci = (int)(c - s_bound[1]);
      ch.kind = KIND_C2;
      ch.rb = div_small(ci, p.inv_cprC2);  // output row-block
      ch.kc = ci - ch.rb * p.cprC2;
      ch.k0 = ch.kc * p.spcC2;
      ch.n = min(p.spcC2, p.sprC2 - ch.k0);
      ch.slot = p.topk;
      const size_t wrow = p.shared_inter / 8;
      ch.w_lo = reinterpret_cast<const uint4 *>(p.shared_down) + (size_t)(ch.rb * 16 + g) * wrow;
      ch.w_hi = ch.w_lo + 8 * wrow;
    }
    return ch;
  };

  // The routing is computed once per CTA, by the first warp that needs it, from the tagged
  // logits (polled until the router's finishers have written them); same inputs, same rule,
  // so every CTA selects the same experts.  The other warps wait on a shared-memory flag.
  auto fetch_routing = [&]() {
    if (claim_or_wait(&s_route_state, lane, err, 1u)) {
      if (lane == 0) trace_cta(p, 3);
      uint16_t *ids_out = blockIdx.x == 0 ? p.ids_out : nullptr;  // CTA 0 reports the routing to the caller
      float *wts_out = blockIdx.x == 0 ? p.wts_out : nullptr;
      if (p.experts <= 128) routing_from_scores<4>(p.logits, p.logits + p.experts, w_ids, w_wts, ids_out, wts_out, p.experts, p.topk, p.routed_scale, epoch, err, lane);
      else routing_from_scores<12>(p.logits, p.logits + p.experts, w_ids, w_wts, ids_out, wts_out, p.experts, p.topk, p.routed_scale, epoch, err, lane);
      if (lane == 0 && blockIdx.x == 0) trace_launch(p, 1);
      if (p.part_out) {
        // keep the slots whose expert this rank holds, in selection order, with the expert's index in the rank's arrays;
        // the queue's B and C1 phases shrink to those slots
        __syncwarp();
        const int id = lane < p.topk ? w_ids[lane] - p.expert_base : -1;
        const float wv = lane < p.topk ? w_wts[lane] : 0.f;
        const bool mine = id >= 0 && id < p.experts_local;
        const unsigned m = __ballot_sync(0xffffffffu, mine);
        __syncwarp();
        if (mine) {
          const int j = __popc(m & ((1u << lane) - 1u));
          w_ids[j] = id;
          w_wts[j] = wv;
        }
        if (lane == 0) {
          const unsigned n = (unsigned)__popc(m);
          s_slots = (int)n;
          s_bound[0] = p.cB0 + n * ((p.cC10 - p.cB0) / (unsigned)p.topk);
          s_bound[1] = s_bound[0] + n * ((p.cC20 - p.cC10) / (unsigned)p.topk);
          s_bound[2] = s_bound[1] + (p.total - p.cC20);
        }
      }
      publish(&s_route_state, lane);
      if (lane == 0) trace_cta(p, 2);
    }
    have_routing = true;
  };

  // A slot's mid vector (slot == topk: the shared expert's), prepared once per CTA by the first warp that needs it.
  auto ensure_mid = [&](int slot) {
    if (!claim_or_wait(&s_mid_state[slot], lane, err, 4u)) return;
    stage_mid_i4(p.mid_cnt + slot, p.mid + (size_t)slot * (p.mid_stride / 2), p.inter, midq + (size_t)slot * midq_bytes, epoch, err, lane);
    publish(&s_mid_state[slot], lane);
  };
  auto ensure_smid = [&]() {
    if (!claim_or_wait(&s_mid_state[p.topk], lane, err, 5u)) return;
    stage_mid_bf16(p.mid_cnt + p.topk, p.mid + (size_t)p.topk * (p.mid_stride / 2), p.shared_inter, smid, epoch, err, lane);
    publish(&s_mid_state[p.topk], lane);
  };

  auto piece_part = [&](const Chunk &ch) { return ch.kind == KIND_R ? p.partR : ch.kind == KIND_A ? p.partA : ch.kind == KIND_B ? p.partB : p.partC2; };
  auto piece_cnt = [&](const Chunk &ch) { return ch.kind == KIND_R ? p.cntR : ch.kind == KIND_A ? p.cntA : ch.kind == KIND_B ? p.cntB : p.cntC2; };
  auto piece_n = [&](const Chunk &ch) { return ch.kind == KIND_R ? p.cprR : ch.kind == KIND_A ? p.cprA : ch.kind == KIND_B ? p.cprB : p.cprC2; };

  // v holds A row g + 8 * (t >> 1) in every lane of a quad half; lanes 0..15 receive rows 0..15
  auto rows_to_lanes = [&](float v) { return __shfl_sync(0xffffffffu, v, ((lane & 7) << 2) + ((lane >> 3) & 1) * 2); };

  // Handing a finished chunk in.  No warp ever waits for another chunk of its row-block: every chunk stores its 16 partial
  // sums and increments the row-block's counter; the warp whose increment completes the row-block finishes it (complete()).
  // arrive() returns the counter's old value in lane 0; the increment's latency is covered by what the caller does before
  // it looks at the value (the next chunk's first requests).
  auto arrive = [&](const Chunk &ch, float v) -> unsigned {
    if (ch.kind == KIND_R && p.r_local) {
      // the 16 chunks of a router row-block are this CTA's 16 first chunks: their sums meet in shared memory, no global
      // round trip lies between the last weight byte of the router and its logits
      if ((t & 1) == 0) s_rpart[warp][g + 8 * (t >> 1)] = v;
      __threadfence_block();
      __syncwarp();
      unsigned old = 0;
      if (lane == 0) old = (unsigned)atomicAdd(&s_rcount, 1);
      return old;
    }
    if (ch.kind == KIND_C1) {
      const float total = rows_to_lanes(v);
      if (lane < 16) st_tagged(p.ys + (size_t)ch.slot * p.hidden + ch.rb * 16 + lane, round_bf16(total), epoch);
      return 0u;
    }
    const int np = piece_n(ch);
    if (np == 1) return epoch - 1u;  // the only chunk of its row-block completes it
    if ((t & 1) == 0) __stcg(piece_part(ch) + ((size_t)ch.rb * np + ch.kc) * 16 + g + 8 * (t >> 1), v);
    __syncwarp();
    unsigned old = 0;
    if (lane == 0) old = arrive_counter(piece_cnt(ch) + ch.rb);
    return old;
  };

  // lanes 0..15 hold the 16 logits of router row-block rb, unrounded (:297): s = 1 / (1 + expf(-logit)) (:379),
  // sel = s + bias (:374), both published per expert
  auto publish_scores = [&](int rb, float logit) {
    if (lane < 16) {
      const int e = rb * 16 + lane;
      const float sc = 1.0f / (1.0f + expf(-logit));
      st_tagged(p.logits + e, sc + p.router_bias[e], epoch);
      st_tagged(p.logits + p.experts + e, sc, epoch);
    }
  };

  auto complete = [&](const Chunk &ch, float v, unsigned old) {
    if (ch.kind == KIND_C1) {
      // without a shared expert the last routed slot finishes the output rows (its own rows are in memory by now: arrive())
      if (p.shared_inter == 0 && ch.slot == p.topk - 1)
        combine_rows(p.ys, p.y, p.hidden, p.topk, false, w_wts, ch.rb, 0.f, epoch, err, lane, nullptr, nullptr);
      return;
    }
    const int np = piece_n(ch);
    old = __shfl_sync(0xffffffffu, old, 0);
    if (ch.kind == KIND_R && p.r_local) {
      if (old + 1u != (unsigned)kFusedWarps) return;
      __threadfence_block();
      float total = 0.f;
      if (lane < 16)
        for (int wi = 0; wi < kFusedWarps; ++wi) total += s_rpart[wi][lane];  // chunk order
      publish_scores(ch.rb, total);
      if (lane == 0) trace_launch(p, 5);
      return;
    }
    if (old + 1u != epoch * (unsigned)np) return;  // another chunk of the row-block is still out
    const float total = np > 1 ? collect_row_block(piece_part(ch) + (size_t)ch.rb * np * 16, np, lane) : rows_to_lanes(v);
    if (ch.kind == KIND_R) {
      publish_scores(ch.rb, total);
      if (lane == 0) trace_launch(p, 5);
      return;
    }
    if (ch.kind == KIND_A || ch.kind == KIND_B) {
      const int row0 = ch.kind == KIND_A ? ch.rb * 8 : (ch.rb - ch.slot * (p.inter / 8)) * 8;
      const unsigned before = publish_mid(total, p.mid + ((size_t)ch.slot * p.mid_stride + row0) / 2, p.mid_cnt + ch.slot, lane);
      if (p.trace && lane == 0) {
        trace_launch(p, ch.kind == KIND_A ? 11 : 12);
        if (ch.kind == KIND_B && before + 1u == epoch * (unsigned)(p.inter / 8)) {  // a slot's mid vector is complete
          if (ch.slot == 0) trace_launch(p, 14);
          if (ch.slot == 3) trace_launch(p, 4);
          if (ch.slot == 5) trace_launch(p, 6);
          if (ch.slot == p.topk - 1) trace_launch(p, 15);
        }
      }
      return;
    }
    // KIND_C2: the shared expert's rows are complete, and with them the output rows
    combine_rows(p.ys, p.y, p.hidden, s_slots, p.shared_inter != 0, w_wts, ch.rb, round_bf16(total), epoch, err, lane, p.part_out,
                 p.shared_out);
    if (lane == 0) trace_launch(p, 13);
  };

  // ---- the first chunk's weights go in flight before anything else: the first pass over the queue is the router and
  // the shared expert's gate/up, which need nothing but x ------------------------------------------------------------
  const unsigned W = gridDim.x * kFusedWarps;
  unsigned c = blockIdx.x * kFusedWarps + warp;
  Chunk cur;
  cur.kind = KIND_NONE;
  const bool early = c < p.cB0 && c < p.total;  // needs no routing
  if (early) {
    cur = decode(c);
    ring_prologue(cur, ring, lane);
  }
  if (tid == 0) trace_cta(p, 4);
  stage_x_both(p.x, xnat, xq.xq, xq.meta, xq.zero, p.hidden, tid);
  if (tid == 0) trace_cta(p, 5);
  __syncthreads();
  if (tid == 0) trace_cta(p, 1);
  if (!early && c < p.total) {
    if (c < p.cC20 || p.part_out) fetch_routing();  // a rank's share: the routing also fixes where C2 starts in the queue
    if (c < s_bound[2]) {
      cur = decode(c);
      ring_prologue(cur, ring, lane);
    }
  }

  // integer form: lanes with (g >> 1) == t supply limb g & 1 of their own scale group (two uint4 per k-block)
  const bool supply = ((g >> 1) == t);
  ImmaLane xl_x;  // x
  xl_x.ptr = supply ? reinterpret_cast<const uint4 *>(xq.xq + t * 64 + (g & 1) * 32) : xq.zero + 4 + (lane & 1);
  xl_x.kb_stride = supply ? 16 : 0;

  int traced = 0, traced_w = 0;
  while (cur.kind != KIND_NONE) {
    // ---- the chunk's weights are in flight; now the activations -------------------------------
    Consumed got;
    const bool tr = p.trace && warp == 0 && lane == 0 && traced < 1;
    if (tr) p.trace[16 + (size_t)blockIdx.x * kTraceSlots + 11] = global_ns();
    const uint4 *w_lo = cur.w_lo + (size_t)cur.k0 * 4 + t, *w_hi = cur.w_hi + (size_t)cur.k0 * 4 + t;
    if (cur.kind == KIND_C1) {
      ensure_mid(cur.slot);
      const unsigned char *mq = midq + (size_t)cur.slot * midq_bytes;
      const uint4 *xp = supply ? reinterpret_cast<const uint4 *>(mq + t * 64 + (g & 1) * 32) : xq.zero + 4 + (lane & 1);
      got = consume_i4(w_lo, w_hi, cur.n, ring, ring_ptr, xp, supply ? 16 : 0, reinterpret_cast<const uint2 *>(mq + (size_t)p.inter * 2),
                       p.ctrl + CTRL_QUEUE, W, lane);
    } else if (cur.kind == KIND_C2) {
      if (!have_routing) fetch_routing();  // the combine needs the routing weights
      ensure_smid();
      got = consume_bf16(w_lo, w_hi, cur.n, ring, ring_ptr, smid + (size_t)cur.k0 * 4 + t, p.ctrl + CTRL_QUEUE, W, lane);
    } else if (cur.kind == KIND_B) {
      got = consume_i4(w_lo, w_hi, cur.n, ring, ring_ptr, xl_x.ptr + (size_t)cur.k0 * xl_x.kb_stride, xl_x.kb_stride,
                       xq.meta + (size_t)cur.k0 * 4, p.ctrl + CTRL_QUEUE, W, lane);
    } else {
      got = consume_bf16(w_lo, w_hi, cur.n, ring, ring_ptr, xnat + (size_t)cur.k0 * 4 + t, p.ctrl + CTRL_QUEUE, W, lane);
    }
    // ---- hand in (without waiting), put the next chunk's weights in flight, then look at the count ----
    if (tr) p.trace[16 + (size_t)blockIdx.x * kTraceSlots + 12] = global_ns(), ++traced;
    const float v = got.v;
    if (p.trace && lane == 0 && traced_w < 1) {  // per warp: when its first chunk was consumed
      p.trace[(size_t)(gridDim.x + 1) * 16 + ((size_t)blockIdx.x * kFusedWarps + warp) * 2] = global_ns();
    }
    const unsigned old = arrive(cur, v);
    c = __shfl_sync(0xffffffffu, got.next, 0);
    Chunk nx;
    nx.kind = KIND_NONE;
    bool completed = false;
    if (c < p.total) {
      if (p.trace && lane == 0) {  // when the queue reaches each phase, and its end
        if (c == p.cB0) trace_launch(p, 7);
        if (c == p.cC10) trace_launch(p, 8);
        if (c == p.cC20) trace_launch(p, 9);
        if (c == p.total - 1) trace_launch(p, 10);
      }
      if (c >= p.cB0 && (c < p.cC20 || p.part_out) && !have_routing) {
        // the routing may depend on the chunk in hand: finish it before waiting
        complete(cur, v, old);
        completed = true;
        fetch_routing();
      }
      if (c < p.cB0 || c < s_bound[2]) {
        nx = decode(c);
        ring_prologue(nx, ring, lane);
      }
    }
    if (!completed) complete(cur, v, old);
    if (p.trace && lane == 0 && traced_w < 1) {  // ... and when the warp was through with it (row-block finished, if it was its finisher)
      p.trace[(size_t)(gridDim.x + 1) * 16 + ((size_t)blockIdx.x * kFusedWarps + warp) * 2 + 1] = global_ns();
      ++traced_w;
    }
    cur = nx;
  }

  // CTA 0 reports the routing to the caller; with a rank's share every CTA may turn out to be the last one, which must
  // know how many slots the launch used
  if (warp == 0 && !have_routing && (blockIdx.x == 0 || p.part_out)) fetch_routing();
  // ---- the last CTA to leave resets the launch-wide counters ------------------------------------
  cp_async_wait<0>();
  if (warp == 0 && lane == 0) trace_cta(p, 6);
  __syncthreads();
  if (tid == 0) {
    trace_cta(p, 7);
    const unsigned epoch_now = p.ctrl[CTRL_EPOCH] + 1u;
    if (p.err_host) __threadfence_system();  // y may lie in host memory
    else __threadfence();
    unsigned old = atomicAdd(p.ctrl + CTRL_EXIT, 1u);
    s_last = old == gridDim.x - 1;
    if (old == gridDim.x - 1) {
      p.ctrl[CTRL_QUEUE] = 0;
      p.ctrl[CTRL_EXIT] = 0;
      p.ctrl[CTRL_EPOCH] = epoch_now;
      if (p.err_host) {  // every CTA's outputs were fenced before its exit count: the host sees them before this word
        *reinterpret_cast<volatile unsigned *>(p.err_host) = __ldcg(p.ctrl + CTRL_ERROR);
        __threadfence_system();
      }
      __threadfence();
      trace_launch(p, 3);
    }
  }
  if (p.part_out) {
    // The counters count over all launches (a row-block is complete at launch number x its chunks).  The slots this launch
    // left out of the queue did not count: the last CTA to leave sets their counters to what a full launch leaves behind.
    __syncthreads();
    if (s_last) {
      const int rb_slot = p.inter / 8;
      for (int i = s_slots * rb_slot + tid; i < p.topk * rb_slot; i += kFusedThreads) p.cntB[i] = epoch * (unsigned)p.cprB;
      for (int j = s_slots + tid; j < p.topk; j += kFusedThreads) p.mid_cnt[j] = epoch * (unsigned)rb_slot;
    }
  }
}

// ---------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------
static int ceil_div(int a, int b) { return (a + b - 1) / b; }

size_t fused_smem_bytes(const blok_moe_weights &w) {
  return (size_t)w.hidden * 2 + imma_stage_bytes(w.hidden) + (size_t)w.topk * ((size_t)w.inter * 2 + (size_t)(w.inter / 32) * 8) +
         (size_t)w.shared_inter * 2 + (size_t)kFusedWarps * kWarpRingBytes;
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
  if (w.experts % 16 || w.topk > kMaxTopk || w.shared_inter % 32 || w.inter % 256 || w.hidden % 256) return BLOK_OK;
  // the routing keeps every candidate in registers, 12 per lane.  (A 32-per-lane instance for up to 1,024 experts made
  // the whole kernel spill: a callee that wants that many registers costs every caller of the kernel its own.)
  if (w.experts > 384) return BLOK_OK;
  // a rank's share of the experts is served through part_out (launch_moe_decode_fused), which relies on the shared
  // expert's last phase to finish the output rows
  if ((w.experts_local != w.experts || w.expert_base != 0) && w.shared_inter == 0) return BLOK_OK;
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
  int tgt[4] = {14, 28, 14, 32};
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
  plan->enabled = true;
  return BLOK_OK;
}

int launch_moe_decode_fused(blok_moe_layer *L, const uint16_t *x, uint16_t *y, uint16_t *ids_out, float *wts_out,
                            cudaStream_t stream, unsigned *err_host, float *part_out, uint16_t *shared_out) {
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
  p.r_local = pl.cprR == kFusedWarps && pl.nrbR <= pl.grid ? 1 : 0;
  p.mid = reinterpret_cast<uint32_t *>(L->f_mid); p.mid_stride = L->f_mid_stride;
  p.mid_cnt = L->f_cntOut + 8;  // [topk + 1] of the 64 spare counters behind the per-row-block ones
  p.ys = reinterpret_cast<uint2 *>(L->f_ys);
  p.partR = L->f_partR; p.partA = L->f_partA; p.partB = L->f_partB; p.partC2 = L->f_partC2;
  p.cntR = L->f_cntR; p.cntA = L->f_cntA; p.cntB = L->f_cntB; p.cntC2 = L->f_cntC2;
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
  p.inv_cprR = 1.0f / pl.cprR; p.inv_cprA = 1.0f / pl.cprA; p.inv_cprB = 1.0f / pl.cprB; p.inv_cprC2 = 1.0f / pl.cprC2;
  p.inv_rbB = 1.0f / (w.inter / 8); p.inv_rbC1 = 1.0f / (w.hidden / 16);
  p.ctrl = L->f_ctrl;
  p.err_host = err_host;
  p.expert_base = w.expert_base; p.experts_local = w.experts_local;
  p.part_out = part_out; p.shared_out = shared_out;
  p.trace = L->f_trace;
  void *args[] = {&p};
  BLOK_CUDA(cudaLaunchCooperativeKernel((const void *)moe_decode_fused_kernel, dim3(pl.grid), dim3(kFusedThreads), args,
                                        pl.smem, stream));
  return launch_status("moe_decode_fused_kernel");
}

}  // namespace blok
