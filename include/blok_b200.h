/*
 * blok_b200 — C ABI of the B200 (sm_100a) implementation of Blok's decode hot path:
 * the W4A16 routed-expert MoE layer over compressed-tensors pack_quantized INT4
 * weights and the MLA decode attention that feeds it.
 *
 * Conventions
 *  - Every function returns an int status: BLOK_OK (0) or a negative BLOK_ERR_*.
 *    Nothing here calls exit(); blok_last_error() gives the message of the last
 *    failure on the calling thread.  (The reference's die(), src/kimi_exec.cu:495,
 *    terminates the process instead.)
 *  - Every data pointer is a DEVICE pointer owned by the caller unless the
 *    parameter comment says "host".  Work is enqueued on `stream`; no call
 *    synchronises unless stated.
 *  - Only *_create functions allocate.  Stateless entry points that need scratch
 *    take a caller-provided workspace and report its size through *_workspace_bytes.
 *  - bf16 values cross the ABI as uint16_t bit patterns (blok_bf16_t).
 *  - INT4 layout (compressed-tensors pack_quantized, the reference's contract at
 *    src/kimi_exec.cu:599-606, decode rule at :311): weight_packed is int32
 *    [rows, cols/8], nibble = q + 8, nibble k of a word (bits 4k..4k+3) is column
 *    8*word + k; weight_scale is bf16 [rows, cols/32]; dequantised weight =
 *    bf16_rn(float(q) * float(scale)).
 */
#ifndef BLOK_B200_H
#define BLOK_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct CUstream_st *blok_stream_t; /* cudaStream_t */
typedef uint16_t blok_bf16_t;

enum {
  BLOK_OK = 0,
  BLOK_ERR_ARG = -1,         /* null pointer, bad size, misaligned pointer */
  BLOK_ERR_SHAPE = -2,       /* shape not supported by the kernels */
  BLOK_ERR_CUDA = -3,        /* a CUDA runtime call failed */
  BLOK_ERR_STATE = -4,       /* handle misuse */
  BLOK_ERR_TIMEOUT = -5,     /* a bounded device-side wait gave up */
  BLOK_ERR_WORKSPACE = -6,   /* workspace too small */
  BLOK_ERR_ROUTE = -7,       /* routed expert id not held by this rank / capacity exceeded */
  BLOK_ERR_COMM = -8         /* NCCL missing or failed; a peer's memory could not be mapped */
};

/* 2: blok_model_config gained prefill_chunk, kv_page_rows and kv_pages (appended).
 * 3: blok_comm_*, blok_moe_ep_*, blok_model_set_comm; blok_model_config gained ep_rank and ep_world (appended). */
#define BLOK_ABI_VERSION 3

/* Message of the last failure on this thread ("" if none). */
const char *blok_last_error(void);
int blok_abi_version(void);
/* Number of kernels this library has launched in this process (all threads).  No
 * counterpart in the reference; the bench reports it. */
long long blok_kernel_launch_count(void);

/* ------------------------------------------------------------------------- */
/* A1  INT4 weights                                                           */
/* ------------------------------------------------------------------------- */

/* Bit-exactness probe: out[r,c] = bf16_rn(float(q[r,c]) * float(scale[r,c/32])),
 * out is bf16 [rows, cols].  Replaces the dequant expression at
 * src/kimi_exec.cu:311-312.  cols % 32 == 0. */
int blok_i4_dequant(const uint32_t *w_packed, const blok_bf16_t *scale, blok_bf16_t *out, int rows, int cols,
                    blok_stream_t stream);

/* y[r] = bf16(sum_c x[c] * dequant(w[r,c])), fp32 accumulation.  Replaces
 * matvec_i4_slice / matvec_i4_bf16_scale_k (src/kimi_exec.cu:688-690, :300-323).
 * x bf16 [cols], y bf16 [rows].  cols % 128 == 0, rows % 16 == 0 use the
 * tensor-core path; other shapes with cols % 32 == 0 use the scalar path. */
int blok_i4_gemv(const uint32_t *w_packed, const blok_bf16_t *scale, const blok_bf16_t *x, blok_bf16_t *y, int rows,
                 int cols, blok_stream_t stream);

/* Same with the reference's own signature: x and y are fp32 buffers holding
 * bf16-valued numbers (src/kimi_exec.cu:688: const float *x, float *y). */
int blok_i4_gemv_f32(const uint32_t *w_packed, const blok_bf16_t *scale, const float *x, float *y, int rows, int cols,
                     blok_stream_t stream);

/* ------------------------------------------------------------------------- */
/* A2-A4  one routed expert (config 0): y = down(SiLU(gate x) * up x)         */
/* ------------------------------------------------------------------------- */

size_t blok_expert_ffn_workspace_bytes(int hidden, int inter);

/* Replaces the per-slot body of the routed-expert loop, src/kimi_exec.cu:853-869
 * (gate and up GEMV, silu_mul_k :253, down GEMV).  x bf16 [hidden], y bf16 [hidden].
 * gate/up packed [inter, hidden/8] + scale [inter, hidden/32]; down packed
 * [hidden, inter/8] + scale [hidden, inter/32].  hidden % 256 == 0, inter % 256 == 0. */
int blok_expert_ffn(const uint32_t *gate_w, const blok_bf16_t *gate_s, const uint32_t *up_w, const blok_bf16_t *up_s,
                    const uint32_t *down_w, const blok_bf16_t *down_s, const blok_bf16_t *x, blok_bf16_t *y,
                    int hidden, int inter, void *workspace, size_t workspace_bytes, blok_stream_t stream);

/* The same expert for callers that cannot allocate device memory when they call
 * (an engine that owns all of HBM through its own pool, a code path that runs with
 * the allocator locked, a host that forbids allocation after start-up).  It has no
 * counterpart in the reference, whose executor allocates freely (src/kimi_exec.cu
 * cudaMalloc per tile).  The intermediate vector lives in a fixed array inside the
 * library (BLOK_STATIC_MAX_INTER bf16 values, 16 KB, held by every GPU that loads
 * the library until the process exits), so there is no workspace argument and no
 * cudaMalloc / cudaFree anywhere on this path.
 *  - inter > BLOK_STATIC_MAX_INTER is rejected with BLOK_ERR_WORKSPACE.
 *  - The first call on each device looks up the array's device address; make that
 *    first call before any stream capture on that device.
 *  - All calls on a device share the one array: two calls whose kernels can overlap
 *    on the GPU (different streams, no dependency between them) race on it.  Calls
 *    on one stream are safe; nothing needs clearing between calls.
 *  - The looked-up address is kept per device for the life of the process.  After
 *    cudaDeviceReset (or any other destruction and re-creation of the device's
 *    primary context) that address is stale: a process that resets a device must not
 *    call this entry point on it afterwards (blok_expert_ffn with a caller workspace
 *    has no such state). */
#define BLOK_STATIC_MAX_INTER 8192
int blok_expert_ffn_static_max_inter(void);
int blok_expert_ffn_static(const uint32_t *gate_w, const blok_bf16_t *gate_s, const uint32_t *up_w,
                           const blok_bf16_t *up_s, const uint32_t *down_w, const blok_bf16_t *down_s,
                           const blok_bf16_t *x, blok_bf16_t *y, int hidden, int inter, blok_stream_t stream);

/* ------------------------------------------------------------------------- */
/* A6/A7/A10  bf16 GEMV, dense SwiGLU MLP, RMSNorm, residual add               */
/* ------------------------------------------------------------------------- */

/* y[t,r] = sum_c w[r,c] * x[t,c] for T <= 8 tokens; y is bf16 [T, rows] (y_f32 == NULL)
 * or unrounded fp32 [T, rows] (y_bf16 == NULL).  Replaces matvec_bf16_k /
 * matvec_bf16_f32_k (src/kimi_exec.cu:272-298).  cols % 8 == 0. */
int blok_bf16_gemv(const blok_bf16_t *w, const blok_bf16_t *x, blok_bf16_t *y_bf16, float *y_f32, int rows, int cols,
                   int T, blok_stream_t stream);

size_t blok_bf16_mlp_workspace_bytes(int hidden, int ffn, int T);

/* y[t] = W_d (SiLU(W_g x[t]) * W_u x[t]); replaces bf16_mlp (src/kimi_exec.cu:674-686)
 * without its running-sum side effect (the caller adds).  T <= 64; more than 8 rows
 * need hidden and ffn to be multiples of 256 and stream each matrix once for all rows
 * (the workspace then also holds the K-split partial sums of the down projection). */
int blok_bf16_mlp(const blok_bf16_t *gate, const blok_bf16_t *up, const blok_bf16_t *down, const blok_bf16_t *x,
                  blok_bf16_t *y, int hidden, int ffn, int T, void *workspace, size_t workspace_bytes,
                  blok_stream_t stream);

/* y[t,i] = bf16(bf16(x[t,i] * rsqrt(mean(x[t]^2) + eps)) * w[i]); in place allowed.
 * Replaces rmsnorm_k (src/kimi_exec.cu:258-270).  x, y bf16 [T, n]. */
int blok_rmsnorm(const blok_bf16_t *x, const blok_bf16_t *w, blok_bf16_t *y, int T, int n, float eps,
                 blok_stream_t stream);

/* x <- bf16(x + t) in place, then y = RMSNorm(x) * w, in one launch: the residual add that ends one block and the
 * norm that opens the next (src/kimi_exec.cu:827 + :829, :877 + :812 of the next layer, :877 + :880 after the last). */
int blok_add_rmsnorm(blok_bf16_t *x, const blok_bf16_t *t, const blok_bf16_t *w, blok_bf16_t *y, int T, int n, float eps,
                     blok_stream_t stream);

/* a[i] = bf16(a[i] + b[i]).  Replaces add_k (src/kimi_exec.cu:248-251). */
int blok_add_bf16(blok_bf16_t *a, const blok_bf16_t *b, long n, blok_stream_t stream);

/* ------------------------------------------------------------------------- */
/* A5  router                                                                 */
/* ------------------------------------------------------------------------- */

size_t blok_router_workspace_bytes(int T, int experts);

/* logits = W_r x (fp32, unrounded), s = sigmoid(logits), sel = s + bias, top-k of
 * sel by repeated argmax (ties to the lowest index, output in descending sel
 * order), w_k = s[id_k] / (sum_k s[id_k] + 1e-20) * routed_scale.  Replaces
 * src/kimi_exec.cu:836-842 (matvec_bf16_f32_k :286, sigmoid_k :377, add_bf16_k
 * :372, router_topk_k :382).  x bf16 [T, hidden]; bias fp32 [experts]; ids uint16
 * [T, topk]; wts fp32 [T, topk].  experts <= 1024, topk <= 32. */
int blok_router(const blok_bf16_t *router_w, const float *bias, const blok_bf16_t *x, int T, int experts, int hidden,
                int topk, float routed_scale, uint16_t *ids, float *wts, void *workspace, size_t workspace_bytes,
                blok_stream_t stream);

/* ------------------------------------------------------------------------- */
/* A4-A6  routed-MoE layer (configs 1 and 2)                                  */
/* ------------------------------------------------------------------------- */

typedef struct blok_moe_weights {
  int hidden;        /* 7168 */
  int inter;         /* 2048, routed expert intermediate size */
  int experts;       /* 384, global expert count (router width) */
  int topk;          /* 8 */
  int shared_inter;  /* 2048; 0 = no shared expert */
  float routed_scale; /* 2.827 */
  const blok_bf16_t *router_w; /* [experts, hidden] */
  const float *router_bias;    /* [experts] fp32 (bf16 checkpoints widen exactly) */
  /* Expert-major arrays of the experts this rank holds, ids [expert_base,
   * expert_base + experts_local): packed [n, out, in/8], scale [n, out, in/32]. */
  int expert_base;
  int experts_local;
  const uint32_t *gate_w;
  const blok_bf16_t *gate_s;
  const uint32_t *up_w;
  const blok_bf16_t *up_s;
  const uint32_t *down_w;
  const blok_bf16_t *down_s;
  const blok_bf16_t *shared_gate; /* [shared_inter, hidden] */
  const blok_bf16_t *shared_up;   /* [shared_inter, hidden] */
  const blok_bf16_t *shared_down; /* [hidden, shared_inter] */
} blok_moe_weights;

typedef struct blok_moe_layer blok_moe_layer_t;

/* Allocates the layer's workspace (for up to max_tokens tokens) on the current
 * device.  The weight pointers are borrowed and must outlive the handle. */
int blok_moe_layer_create(const blok_moe_weights *weights, int max_tokens, blok_moe_layer_t **out);
int blok_moe_layer_destroy(blok_moe_layer_t *layer);

/* Batch-1 decode layer: y = bf16(bf16(sum_k w_k * expert_k(x)) + shared(x)).
 * Replaces the MoE branch of the layer body, src/kimi_exec.cu:836-875, with the
 * expert ids kept on the device (no host copy as at :844).  x, y bf16 [hidden];
 * ids_out (uint16 [topk]) and wts_out (fp32 [topk]) may be NULL.  All experts
 * must be local (experts_local == experts). */
int blok_moe_decode(blok_moe_layer_t *layer, const blok_bf16_t *x, blok_bf16_t *y, uint16_t *ids_out, float *wts_out,
                    blok_stream_t stream);

/* Batched layer (config 2): x, y bf16 [T, hidden], T <= max_tokens of the handle.
 * Tokens are permuted by expert, every touched expert's INT4 weights are streamed
 * once through a grouped W4A16 GEMM, outputs are combined per token with the
 * routing weights and the shared expert is added: the arithmetic of
 * src/kimi_exec.cu:836-877 for each token.  ids_out uint16 [T, topk] and wts_out
 * fp32 [T, topk] may be NULL.  All experts must be local. */
int blok_moe_batched(blok_moe_layer_t *layer, const blok_bf16_t *x, int T, blok_bf16_t *y, uint16_t *ids_out,
                     float *wts_out, blok_stream_t stream);

/* The expert half of the batched layer on its own, the building block of expert
 * parallelism: N assignments, assignment a = (row x_index[a] of x, local expert
 * expert_local[a] in [0, experts_local)); y[a, :] = bf16(expert(x_row)) (unweighted;
 * the owner of the token applies the routing weight, as expert_accum_k :399 does).
 * x_index NULL means row a.  N <= max_tokens * topk of the handle. */
int blok_moe_experts_grouped(blok_moe_layer_t *layer, const blok_bf16_t *x, const int *x_index, const int *expert_local,
                             int N, blok_bf16_t *y, blok_stream_t stream);

/* The shared expert for T tokens: out[t] = bf16(W_d(SiLU(W_g x[t]) * W_u x[t])), bf16_mlp
 * (src/kimi_exec.cu:674-686, call site :872-875) without its running-sum side effect.
 * It shares no scratch with blok_moe_experts_grouped: the one exception to "calls on a
 * handle are not concurrent" is that these two may run at the same time on two streams
 * (the expert-parallel layer overlaps the shared expert with the exchange that way). */
int blok_moe_shared(blok_moe_layer_t *layer, const blok_bf16_t *x, int T, blok_bf16_t *out, blok_stream_t stream);

/* out[t] = bf16(bf16(sum_k wts[t,k] * y_assign[t*topk + k]) + shared[t]) in slot order
 * (expert_accum_k :399, round_bf16_k :404, add_k :248); shared may be NULL. */
int blok_moe_combine(const blok_bf16_t *y_assign, const float *wts, const blok_bf16_t *shared, int T, int topk, int hidden,
                     blok_bf16_t *out, blok_stream_t stream);

/* One token through a layer whose handle holds a RANGE of the experts (experts_local < experts): the router and the
 * shared expert run whole, of the selected experts only those in [expert_base, expert_base + experts_local), in the same
 * single launch as blok_moe_decode.  part[hidden] (fp32) = sum over those experts of wts_k * bf16(expert_k(x)),
 * unrounded; shared_out[hidden] (bf16) = the shared expert's output.  Summing `part` over the ranks that together hold
 * every expert, rounding to bf16 and adding shared_out gives blok_moe_decode's y up to the order of the fp32 sum
 * (expert_accum_k :399 adds in selection order; here each rank adds its own experts in selection order first).
 * ids_out / wts_out (may be NULL) receive the full routing.  Needs a shared expert and a layer the single-launch kernel
 * serves: blok_moe_layer_has_partial tells (1 / 0); BLOK_ERR_STATE otherwise. */
int blok_moe_decode_partial(blok_moe_layer_t *layer, const blok_bf16_t *x, float *part, blok_bf16_t *shared_out,
                            uint16_t *ids_out, float *wts_out, blok_stream_t stream);
int blok_moe_layer_has_partial(blok_moe_layer_t *layer);

/* Synchronises `stream` and reports whether a device-side wait of an earlier
 * blok_moe_decode on this handle gave up (BLOK_ERR_TIMEOUT; the handle is reset
 * and stays usable).  The reference has no such state: its kernels never wait
 * on one another (src/kimi_exec.cu launches are all on the default stream). */
int blok_moe_layer_check(blok_moe_layer_t *layer, blok_stream_t stream);

/* Test hook (host-side fault injection; nothing faults or hangs on the device): stores `code` in the handle's device
 * error word exactly as a wait that gave up would, so that the reporting path (blok_moe_layer_check, blok_model_check,
 * blok_moe_decode_host) can be exercised. */
int blok_moe_layer_debug_set_error(blok_moe_layer_t *layer, unsigned code, blok_stream_t stream);

/* Diagnostics (no counterpart in the reference): with BLOK_MLA_TRACE=1 in the environment at the first attention
 * launch, CTA (0, 0) of the attention core records, for its first 64 tiles of 64 tokens, 16 slots of nanosecond time
 * stamps per tile (buffer free, tile landed, scores issued, scores seen, probabilities handed over, P.C issued, ...: the
 * kernel's source lists them).  Copies up to max_entries of them to host_out after a device synchronise; returns the count (0: tracing off). */
int blok_mla_attend_trace(long long *host_out, int max_entries);

/* Diagnostics (no counterpart in the reference): when the handle was created with
 * the environment variable BLOK_MOE_TRACE=1, the fused decode kernel records
 * nanosecond time stamps: 16 launch-wide slots, then 16 slots per CTA.  Copies up to max_entries of
 * them to host_out after a device synchronise; returns the count (0 = tracing off). */
int blok_moe_layer_trace(blok_moe_layer_t *layer, long long *host_out, int max_entries);

/* The same layer with HOST buffers: copies x_host (bf16 [hidden]) to the device,
 * runs blok_moe_decode, copies the result to y_host and synchronises `stream`
 * before returning.  This is the call shape of the reference's own boundary,
 * where activations enter and leave through host memory per token
 * (src/kimi_exec.cu:651-655 embed, :728-730 sampled id); pinned host memory
 * makes the two copies asynchronous with respect to the host. */
int blok_moe_decode_host(blok_moe_layer_t *layer, const blok_bf16_t *x_host, blok_bf16_t *y_host,
                         blok_stream_t stream);

/* ------------------------------------------------------------------------- */
/* Expert parallelism (config 2 at 2/4/8 GPUs; the model of config 4)          */
/* ------------------------------------------------------------------------- */

/* The reference runs on one GPU and has no collective (src/kimi_exec.cu has no multi-GPU code), so nothing in this
 * section replaces a reference function; per token the arithmetic is still :836-877.  One process per GPU; expert e
 * lives on rank e / (experts / world). */
typedef struct blok_comm blok_comm_t;
#define BLOK_COMM_ID_BYTES 128
/* HOST: fills id_out (BLOK_COMM_ID_BYTES bytes) with a fresh NCCL unique id.  One rank calls it and hands the bytes to
 * the others by whatever means the launcher offers (a file, an environment, a torch.distributed broadcast). */
int blok_comm_unique_id(void *id_out);
/* Collective over all `world` ranks: joins the communicator on the CURRENT device.  NCCL is resolved at run time
 * (dlopen of libnccl.so.2, or the path in BLOK_NCCL_LIB), so single-GPU users of the library need none. world == 1
 * needs no id and no NCCL.  BLOK_ERR_COMM when NCCL is missing or refuses. */
int blok_comm_create(const void *unique_id, int rank, int world, blok_comm_t **out);
int blok_comm_destroy(blok_comm_t *comm);
int blok_comm_rank(const blok_comm_t *comm);
int blok_comm_world(const blok_comm_t *comm);
/* BLOK_ERR_COMM if NCCL has reported an asynchronous error on the communicator (a peer that died, a deadline). */
int blok_comm_check(blok_comm_t *comm);
/* In-place sum over the ranks of n floats on the device, and a broadcast of bytes from `root`: the two collectives
 * the sharded model needs (one all-reduce per MoE layer).  Up to 262,144 floats (n a multiple of 4, buf 16-byte
 * aligned) the all-reduce is two launches of the library's own kernels over peer memory: every rank stores its
 * vector into its slot of every rank's region over NVLink, then a flag with the call number; every rank adds the slots
 * in rank order, so all ranks end with the same bits.  No library call, no host synchronisation, replayable from a CUDA
 * graph (the call number lives on the device).  A peer that never signals ends the bounded wait and is reported by
 * blok_comm_check (BLOK_ERR_TIMEOUT).  Longer vectors, or BLOK_COMM_ALLREDUCE=nccl in the environment: ncclAllReduce. */
int blok_comm_all_reduce_f32(blok_comm_t *comm, float *buf, long n, blok_stream_t stream);
int blok_comm_broadcast(blok_comm_t *comm, void *buf, long bytes, int root, blok_stream_t stream);

/* The batched layer (blok_moe_batched) with the experts split over the ranks.  `weights` describes THIS rank's shard:
 * experts_local = experts / world, expert_base = rank * experts_local, the expert arrays holding only those experts;
 * router and shared expert are replicated.  max_tokens bounds the tokens a rank brings to one pass.
 * Collective: every rank creates its handle at the same point (the ranks map one another's receive buffers:
 * world * max_tokens * topk rows of hidden bf16, twice, per rank). */
typedef struct blok_moe_ep blok_moe_ep_t;
int blok_moe_ep_create(blok_comm_t *comm, const blok_moe_weights *weights, int max_tokens, blok_moe_ep_t **out);
int blok_moe_ep_destroy(blok_moe_ep_t *ep);
/* One pass; every rank must call it the same number of times (T may differ per rank and may be 0).  x, y bf16
 * [T, hidden] are this rank's tokens; ids_out uint16 [T, topk] (global expert ids) and wts_out fp32 [T, topk] may be
 * NULL.  Dispatch and combine run inside the library's kernels over peer memory (plain stores and loads over NVLink,
 * flags that carry the pass number); nothing synchronises with the host.  y[t] = bf16(bf16(sum_k w_k expert_k(x[t]))
 * + shared(x[t])), slot order as :868-871, :684. */
int blok_moe_ep_forward(blok_moe_ep_t *ep, const blok_bf16_t *x, int T, blok_bf16_t *y, uint16_t *ids_out, float *wts_out,
                        blok_stream_t stream);
/* Synchronises `stream`; BLOK_ERR_TIMEOUT if a bounded wait for a peer gave up in an earlier pass (the message says
 * which), BLOK_ERR_ROUTE if more rows arrived than the receive buffer holds, BLOK_ERR_COMM for an NCCL error. */
int blok_moe_ep_check(blok_moe_ep_t *ep, blok_stream_t stream);
/* HOST out[4] after synchronising `stream`, for the last pass: assignments this rank sent, of those to other ranks,
 * rows this rank received, tiles its grouped GEMM ran. */
int blok_moe_ep_stats(blok_moe_ep_t *ep, long long *host_out4, blok_stream_t stream);
/* The exchange plan of one rank, on the HOST (no GPU needed), from the count table every rank holds after the
 * histograms were gathered: table int32 [world, experts], table[s, g] = assignments rank s sends to expert g.  It runs
 * the same code as the plan kernel of blok_moe_ep_forward and exists so that this arithmetic can be exercised among
 * CPU ranks.  Outputs: send_base [experts] = the row, in the owner's receive buffer, of this rank's first assignment
 * to expert g (the owner's buffer is ordered by expert, then by source rank); as owner: counts [experts/world],
 * offsets [experts/world + 1], and the tiles (<= 64 rows of one expert) of its grouped GEMM, at most max_tiles of them.
 * BLOK_ERR_ROUTE when more than cap_rows rows would arrive. */
int blok_ep_plan_host(const int *table, int world, int experts, int rank, long cap_rows, int max_tiles, int *send_base, int *counts,
                      int *offsets, int *tile_expert, int *tile_start, int *tile_count, int *num_tiles);

/* Measurement aid: with profiling on, a pass records a CUDA event between its phases; blok_moe_ep_phase_ms waits for
 * the last pass and returns HOST out[6], milliseconds on the device: routing; counts + plan + dispatch; shared expert;
 * waiting for the other ranks' rows; the grouped expert GEMM; flags + combine (which waits for the owners). */
int blok_moe_ep_profile(blok_moe_ep_t *ep, int on);
int blok_moe_ep_phase_ms(blok_moe_ep_t *ep, float *host_out6);

/* ------------------------------------------------------------------------- */
/* A8-A10  MLA decode attention (config 3)                                    */
/* ------------------------------------------------------------------------- */

typedef struct blok_mla_weights {
  int hidden;   /* 7168 */
  int heads;    /* 64 */
  int qk_nope;  /* 128 */
  int qk_rope;  /* 64 */
  int v_head;   /* 128 */
  int q_rank;   /* 1536 */
  int kv_rank;  /* 512 */
  float rms_eps;          /* 1e-5 (src/kimi_exec.cu:183) */
  float rope_theta;       /* 50000 */
  float yarn_factor;      /* 64 in the reference (:184), 32 in the benchmark configuration */
  float yarn_beta_fast;   /* 32 */
  float yarn_beta_slow;   /* 1 */
  float yarn_original_ctx; /* 4096 */
  float yarn_mscale_all_dim; /* 1 */
  const blok_bf16_t *q_a;      /* [q_rank, hidden] */
  const blok_bf16_t *q_a_ln;   /* [q_rank] */
  const blok_bf16_t *q_b;      /* [heads*(qk_nope+qk_rope), q_rank] */
  const blok_bf16_t *kv_a;     /* [kv_rank+qk_rope, hidden] (kv_a_proj_with_mqa) */
  const blok_bf16_t *kv_a_ln;  /* [kv_rank] */
  const blok_bf16_t *kv_b;     /* [heads*(qk_nope+v_head), kv_rank] */
  const blok_bf16_t *o;        /* [hidden, heads*v_head] */
} blok_mla_weights;

typedef struct blok_mla_layer blok_mla_layer_t;

/* Allocates the layer's workspace for up to max_batch (<= 64) sequences, or tokens of a
 * prefill chunk, and up to max_ctx cached tokens each, and a transposed copy of the W_UK
 * half of kv_b. */
int blok_mla_layer_create(const blok_mla_weights *weights, int max_batch, int max_ctx, blok_mla_layer_t **out);
int blok_mla_layer_destroy(blok_mla_layer_t *layer);
/* Rebuilds what create derived from the weights (the transposed W_UK copy) after the caller has overwritten kv_b in
 * place.  Synchronises the device. */
int blok_mla_layer_refresh(blok_mla_layer_t *layer);

/* One decode step of the attention block for B sequences, one new token each.
 * Replaces src/kimi_exec.cu:813-826 (q_a -> norm -> q_b, kv_a -> norm, RoPE,
 * KV store, tiled_attention :692-716, o_proj) in the absorbed form over a bf16
 * latent cache: row [b, t] of `cache` is (normed c_kv [kv_rank], roped k_pe
 * [qk_rope]), the state the reference itself holds in bf16-valued form.
 *   n        bf16 [B, hidden]  the normed hidden state (output of the input RMSNorm, :812)
 *   cache    bf16 [B, ctx_stride, kv_rank+qk_rope]; this call WRITES row ctx_len[b]
 *   ctx_len  int32 [B] on the device: tokens already cached; also the new token's position
 *   out      bf16 [B, hidden]  o_proj output (the caller adds the residual, :827)
 * Attention covers positions 0..ctx_len[b] inclusive.  ctx_len[b] < ctx_stride. */
int blok_mla_decode(blok_mla_layer_t *layer, const blok_bf16_t *n, blok_bf16_t *cache, long ctx_stride,
                    const int *ctx_len, int B, blok_bf16_t *out, blok_stream_t stream);

/* The cache positions live on the device (ctx_len), so a position outside a sequence's rows (ctx_len[b] >= ctx_stride;
 * paged: beyond table_stride pages) cannot be refused before the launch.  The kernels then skip the store of that row,
 * keep the attention inside the rows and record the entry; this call synchronises `stream` and returns BLOK_ERR_SHAPE
 * once for it.  (The reference dies on the host at its capacity check, src/kimi_exec.cu:205.)  The page numbers in a
 * block table are the caller's: they are not checked against the pool. */
int blok_mla_layer_check(blok_mla_layer_t *layer, blok_stream_t stream);

/* The attention core alone, for measurement and parity: q bf16 [B, heads,
 * kv_rank+qk_rope] (absorbed nope part, then roped part), seq_len int32 [B] on the
 * device (tokens to attend to), o_lat bf16 [B, heads, kv_rank] =
 * softmax(q . cache^T * scale) . cache[:, :kv_rank].  Replaces the score / max /
 * sum / accumulate kernels at src/kimi_exec.cu:414-475. */
int blok_mla_attend(blok_mla_layer_t *layer, const blok_bf16_t *q, const blok_bf16_t *cache, long ctx_stride,
                    const int *seq_len, int B, float softmax_scale, blok_bf16_t *o_lat, blok_stream_t stream);

/* A prefill chunk: T consecutive tokens of ONE sequence through the attention block in one call, instead of the
 * reference's token-by-token prompt replay (src/kimi_exec.cu:885-886).  Token i sits at position first_pos[0] + i;
 * all T latent rows are appended first, then token i attends to positions 0..first_pos[0]+i (causal), which is what
 * T calls of blok_mla_decode would compute.
 *   n          bf16 [T, hidden]        cache   bf16 [ctx_cap, kv_rank+qk_rope], this sequence's rows
 *   first_pos  int32 [1] on the device: tokens already cached; first_pos[0] + T <= ctx_cap is the caller's duty
 *   out        bf16 [T, hidden]        T <= max_batch of the handle (<= 64) */
int blok_mla_prefill(blok_mla_layer_t *layer, const blok_bf16_t *n, blok_bf16_t *cache, long ctx_cap, const int *first_pos,
                     int T, blok_bf16_t *out, blok_stream_t stream);

/* blok_mla_decode over a PAGED latent cache (the reference's KvCache, src/kimi_exec.cu:192-238, holds one contiguous
 * region per layer and refuses sequences past its capacity at :205; pages let sequences of different lengths share
 * one pool).  pool is bf16 [pages, page_rows, kv_rank+qk_rope]; page_rows is a multiple of 32.  block_table is int32
 * [slots, table_stride] on the device: entry [s, j] is the page holding rows [j*page_rows, (j+1)*page_rows) of the
 * sequence in slot s.  slot_of int32 [B] (device) names the slot of batch entry b; NULL means slot b.  Several
 * entries may name the same slot with consecutive ctx_len values: that is a prefill chunk of that sequence.
 * The page of row ctx_len[b] must already be in the table (blok_kv_pages_reserve does that on the host). */
int blok_mla_decode_paged(blok_mla_layer_t *layer, const blok_bf16_t *n, blok_bf16_t *pool, const int *block_table,
                          const int *slot_of, int table_stride, int page_rows, const int *ctx_len, int B,
                          blok_bf16_t *out, blok_stream_t stream);

/* blok_mla_attend over the same paged pool. */
int blok_mla_attend_paged(blok_mla_layer_t *layer, const blok_bf16_t *q, const blok_bf16_t *pool, const int *block_table,
                          const int *slot_of, int table_stride, int page_rows, const int *seq_len, int B,
                          float softmax_scale, blok_bf16_t *o_lat, blok_stream_t stream);

/* The softmax scale the layer uses: (qk_nope+qk_rope)^-1/2 * mscale^2, mscale =
 * 0.1 * mscale_all_dim * ln(yarn_factor) + 1 (src/kimi_exec.cu:428-429). */
float blok_mla_softmax_scale(const blok_mla_weights *weights);

/* ------------------------------------------------------------------------- */
/* Paged latent cache: host-side page bookkeeping                              */
/* ------------------------------------------------------------------------- */

/* Which pages of a pool every sequence slot holds.  The reference's KvCache (src/kimi_exec.cu:192-238) gives each
 * layer one contiguous region and dies when a sequence outgrows it (:205); here sequences of different lengths draw
 * pages from one pool and return them when they finish.  A page number addresses the same page of every layer's
 * pool, so one table serves all layers.  The handle is host memory only: create, reserve, release and fork make no
 * CUDA call and work without a GPU. */
typedef struct blok_kv_pages blok_kv_pages_t;

/* n_pages pages of page_rows rows (a multiple of 32); `slots` sequences of at most table_stride pages each. */
int blok_kv_pages_create(int n_pages, int page_rows, int slots, int table_stride, blok_kv_pages_t **out);
int blok_kv_pages_destroy(blok_kv_pages_t *pages);
/* Grows the slot's reservation to cover n_rows rows (never shrinks).  BLOK_ERR_WORKSPACE when the pool has too few
 * free pages, BLOK_ERR_SHAPE when n_rows exceeds table_stride * page_rows; the reservation is unchanged then. */
int blok_kv_pages_reserve(blok_kv_pages_t *pages, int slot, long n_rows);
/* Returns the slot's pages to the pool (a page shared through fork goes back when its last holder releases it). */
int blok_kv_pages_release(blok_kv_pages_t *pages, int slot);
/* Lets the empty slot dst share the first n_rows rows (whole pages) of slot src: a common prompt prefix is cached
 * once.  Rows past n_rows of dst go to pages of its own (reserve). */
int blok_kv_pages_fork(blok_kv_pages_t *pages, int src_slot, int dst_slot, long n_rows);
int blok_kv_pages_free_count(const blok_kv_pages_t *pages);
/* Rows the slot's reservation covers. */
long blok_kv_pages_rows(const blok_kv_pages_t *pages, int slot);
/* HOST pointer to the table, int32 [slots, table_stride]; entries past a slot's reservation are 0. */
const int *blok_kv_pages_table(const blok_kv_pages_t *pages);
/* Copies the table to device_table (int32 [slots, table_stride]) on `stream` if it changed since the last upload. */
int blok_kv_pages_upload(blok_kv_pages_t *pages, int *device_table, blok_stream_t stream);

/* ------------------------------------------------------------------------- */
/* A11  embedding fetch and greedy sampler                                    */
/* ------------------------------------------------------------------------- */

/* x[t, :] = table[ids[t], :].  Replaces embed_token (src/kimi_exec.cu:651-655); ids
 * are uint32 on the device and must be < vocab (rows of out-of-range ids are left
 * untouched; the host checks prompt ids as the reference does at :552). */
int blok_embed(const blok_bf16_t *table, const uint32_t *ids, int vocab, int hidden, int T, blok_bf16_t *x,
               blok_stream_t stream);

size_t blok_lm_head_workspace_bytes(int vocab, int T);

/* ids[t] = argmax_v bf16(sum_c W[v,c] n[t,c]), the lowest id winning ties.  Replaces
 * sample_lm_head / argmax_k (src/kimi_exec.cu:718-734, :477-493).  ids stay on the
 * device.  T <= 64; more than 8 rows need vocab % 16 == 0 and hidden % 256 == 0 and
 * read the table once for all rows. */
int blok_lm_head_argmax(const blok_bf16_t *w, const blok_bf16_t *n, int vocab, int hidden, int T, uint32_t *ids,
                        void *workspace, size_t workspace_bytes, blok_stream_t stream);

/* ------------------------------------------------------------------------- */
/* A11/A12  whole model: decode step and greedy generation (config 4)          */
/* ------------------------------------------------------------------------- */

typedef struct blok_model_config {
  int layers;        /* 61 */
  int first_dense;   /* 1: layers [0, first_dense) use the dense FFN (src/kimi_exec.cu:176, :831) */
  int hidden;        /* 7168 */
  int vocab;         /* 163840 */
  int dense_inter;   /* 18432 */
  int inter;         /* 2048 */
  int experts;       /* 384 */
  int topk;          /* 8 */
  int shared_inter;  /* 2048 */
  float routed_scale; /* 2.827 */
  int heads, qk_nope, qk_rope, v_head, q_rank, kv_rank; /* 64, 128, 64, 128, 1536, 512 */
  float rms_eps;       /* 1e-5, every per-layer norm */
  float final_rms_eps; /* 1e-5 in the reference (:880 uses RMS_EPS); 1e-6 in the benchmark configuration */
  float rope_theta, yarn_factor, yarn_beta_fast, yarn_beta_slow, yarn_original_ctx, yarn_mscale_all_dim;
  int max_batch;     /* <= 64 sequences per step */
  int max_ctx;       /* tokens of latent cache per sequence and layer */
  uint32_t eos_id;   /* 163586 (:186) */
  int prefill_chunk; /* 0: the prompt is replayed token by token as in the reference (:886); 1..64: prompts go
                        through blok_model_prefill in chunks of this many tokens */
  int kv_page_rows;  /* 0: every sequence owns max_ctx rows of every layer's cache (the reference's KvCache, :192-238);
                        a multiple of 32: the layers' caches are pools of pages of this many rows, shared by the
                        max_batch resident sequences (slots) through one page table */
  int kv_pages;      /* pages per layer's pool when kv_page_rows > 0 */
  int ep_rank;       /* expert parallelism: with ep_world > 1 this handle is rank ep_rank of ep_world processes, one per GPU; */
  int ep_world;      /* it holds experts [ep_rank, ep_rank + 1) * experts / ep_world of every MoE layer and everything else in
                        full.  0 or 1: the whole model on this GPU.  Needs blok_model_set_comm before the first step. */
} blok_model_config;

typedef struct blok_model blok_model_t;

/* Fills cfg with the reference's constants (src/kimi_exec.cu:176-186). */
void blok_model_default_config(blok_model_config *cfg);

/* Builds a model with seeded synthetic weights on the current device (INT4 words
 * uniform, scales |N(0,0.003)|, bf16 weights N(0,0.006), router bias N(0,0.01), norm
 * weights 1).  Stands in for the checkpoint loader of the reference (:736-778). */
int blok_model_create_synthetic(const blok_model_config *cfg, uint64_t seed, blok_model_t **out);
int blok_model_destroy(blok_model_t *model);

/* Device pointer and byte size of a weight tensor, for tests and loaders.  layer = -1
 * for "embed_tokens", "norm", "lm_head"; per layer: "input_layernorm",
 * "post_attention_layernorm", "q_a_proj", "q_a_layernorm", "q_b_proj", "kv_a_proj_with_mqa",
 * "kv_a_layernorm", "kv_b_proj", "o_proj", dense "gate_proj"/"up_proj"/"down_proj", MoE
 * "router", "router_bias", "gate_w", "gate_s", "up_w", "up_s", "down_w", "down_s",
 * "shared_gate", "shared_up", "shared_down" (the slot names of the reference's index). */
int blok_model_tensor(blok_model_t *model, int layer, const char *name, void **ptr, size_t *bytes);

/* The configuration the model was created with. */
int blok_model_get_config(blok_model_t *model, blok_model_config *cfg);

/* The device buffer that holds, after a step or a prefill chunk has run on its stream, the final-normed hidden states
 * the sampler read (src/kimi_exec.cu:880-881): bf16 [rows used by that call, hidden], row b = sequence b of the step (or
 * token b of the chunk).  *rows is the buffer's capacity in rows.  For parity checks; valid until the next call. */
int blok_model_hidden(blok_model_t *model, const blok_bf16_t **ptr, int *rows);

/* After weights were overwritten in place through blok_model_tensor: rebuilds the copies derived from them at
 * creation (each layer's transposed W_UK). */
int blok_model_refresh_derived(blok_model_t *model);

/* Loads a materialised checkpoint into the model's resident tensors.  `index_path` is the text index
 * "blok-runtime-index-v1" written by the reference's scripts/model_fetch.py:113-127 (one line of 14 fields per
 * tensor: name role layer expert slot dtype shape off bytes align data data_bytes file).  Replaces runtime_index
 * (src/kimi_exec.cu:559-581) and validate_forward_contract (:736-778) with the shapes taken from the model's
 * configuration, and the reference's per-token tile reads with ONE read of every tensor: pread of the byte range
 * [data, data + data_bytes) of `file`, staged through pinned memory into HBM (routed experts into their slice of the
 * expert-major arrays, the router's bf16 correction bias widened to fp32).  Any missing tensor, wrong type, shape,
 * byte count or extent is an error and names the tensor. */
int blok_model_load_index(blok_model_t *model, const char *index_path);

/* The same checks without a model or a GPU: parses the index and verifies the forward contract for cfg.  Returns the
 * number of tensors the model would load and their total bytes. */
int blok_index_validate(const char *index_path, const blok_model_config *cfg, long *n_tensors, unsigned long long *n_bytes);

/* Expert parallelism (config 4 over the GPUs of a node; the reference is a single-GPU program and has no counterpart).
 * Every rank creates its handle with the same configuration and seed apart from ep_rank (the synthetic expert tensors
 * of a rank are the slices of the unsharded tensors), gives it the communicator, and then makes the SAME calls with
 * the same token ids: attention, router, shared expert, embedding and sampler are replicated, so all ranks agree on
 * the routing and on the next token without talking; per MoE layer each rank runs the selected experts it holds and
 * ONE all-reduce (rows x hidden floats) adds the weighted sums, which are then rounded as at :871 and :684.
 * blok_model_tensor returns a rank's shard for the expert tensors.  Steps are replayed from a CUDA graph that
 * holds the all-reduces as well; BLOK_MODEL_GRAPH=0 in the environment keeps every launch eager. */
int blok_model_set_comm(blok_model_t *model, blok_comm_t *comm);

/* Synchronises `stream` and reports, once, whether any layer's bounded device-side wait gave up since the last check
 * (BLOK_ERR_TIMEOUT), a decode position lay outside a cache (BLOK_ERR_SHAPE) or the communicator failed (BLOK_ERR_COMM).
 * blok_model_generate and blok_model_generate_many end with this check: tokens are not returned after such an event.
 * Callers that drive blok_model_step themselves call it where they synchronise anyway. */
int blok_model_check(blok_model_t *model, blok_stream_t stream);

/* Test hook: blok_moe_layer_debug_set_error on the MoE layer `layer` of the model. */
int blok_model_debug_set_layer_error(blok_model_t *model, int layer, unsigned code, blok_stream_t stream);

/* Forgets all cached tokens (positions restart at 0). */
int blok_model_reset(blok_model_t *model);

/* One decode step for B sequences: ids uint32 [B] on the device are embedded, run
 * through every layer at each sequence's current position (appending to the latent
 * caches), and next_ids [B] receives the greedy choice.  Replaces the `run` lambda,
 * src/kimi_exec.cu:801-884.  Positions advance by one. */
int blok_model_step(blok_model_t *model, const uint32_t *ids, int B, uint32_t *next_ids, blok_stream_t stream);

/* Prompt processing for sequence 0 in chunks instead of the reference's token-by-token replay (src/kimi_exec.cu:
 * 885-886): ids uint32 [n] on the device are the next n tokens of the sequence.  Each chunk of up to prefill_chunk
 * tokens runs every layer once: the attention block as a causal chunk (blok_mla_prefill), the routed experts through
 * the grouped GEMM (blok_moe_batched; token by token when the layer's sizes do not fit that kernel).  Only the last
 * token is sampled: next_id uint32 [1] on the device.  The position of sequence 0 advances by n.  The result is what
 * n calls of blok_model_step would give, up to the summation order of the batched kernels.  Needs prefill_chunk >= 1. */
int blok_model_prefill(blok_model_t *model, const uint32_t *ids, int n, uint32_t *next_id, blok_stream_t stream);

/* The paged model (kv_page_rows > 0): batch entry b of a step is the resident sequence in slot slots[b] (HOST array of
 * B distinct slots in [0, max_batch)), so a step can run any subset of the resident sequences.  Before launching, the
 * pages for each sequence's next row are reserved; when the pool cannot supply them the call returns
 * BLOK_ERR_WORKSPACE and launches nothing.  ids / next_ids uint32 [B] on the device, in batch order.
 * blok_model_step on a paged model is this call with slots 0..B-1. */
int blok_model_step_slots(blok_model_t *model, const int *slots, int B, const uint32_t *ids, uint32_t *next_ids,
                          blok_stream_t stream);
/* blok_model_prefill for the sequence in `slot` of a paged model (a dense model accepts slot 0 only). */
int blok_model_prefill_slot(blok_model_t *model, int slot, const uint32_t *ids, int n, uint32_t *next_id,
                            blok_stream_t stream);
/* Ends the sequence in `slot`: its position returns to 0 and, on a paged model, its pages go back to the pool. */
int blok_model_slot_release(blok_model_t *model, int slot, blok_stream_t stream);
/* Tokens cached for the sequence in `slot` (host-side count), and free pages of the pool (-1 on a dense model). */
long blok_model_slot_length(blok_model_t *model, int slot);
int blok_model_free_pages(blok_model_t *model);

/* ------------------------------------------------------------------------- */
/* Continuous batching: host-side scheduler                                    */
/* ------------------------------------------------------------------------- */

/* Decides, iteration by iteration, which queued request enters which sequence slot and which slots step.  Every
 * sequence follows the reference's own rule (src/kimi_exec.cu:885-890: prompt, then one token per iteration until EOS
 * or max_new tokens; EOS is not emitted); up to `slots` of them run side by side over a pool of n_pages pages of
 * page_rows rows.  Admission is in arrival order and reserves a request's whole budget (prompt + max_new rows), so a
 * running sequence never finds the pool empty and none is evicted.  Host memory only: no CUDA call, works without a GPU. */
typedef struct blok_batcher blok_batcher_t;
int blok_batcher_create(int slots, int n_pages, int page_rows, int max_ctx, blok_batcher_t **out);
int blok_batcher_destroy(blok_batcher_t *batcher);
/* Queues a request; ids count up from 0.  BLOK_ERR_SHAPE when n_prompt + max_new exceeds max_ctx (the reference's
 * check, :784), BLOK_ERR_WORKSPACE when the pool could never hold it. */
int blok_batcher_submit(blok_batcher_t *batcher, int n_prompt, int max_new, int *request_id);
/* The next iteration: decode_slots[0..n_decode) are the running sequences, which step once; admit_slots[i] /
 * admit_requests[i], i < n_admit, are the requests that enter now (the caller prefills their prompts).  All arrays
 * hold `slots` ints.  Every slot listed must be answered with blok_batcher_token before the next plan. */
int blok_batcher_plan(blok_batcher_t *batcher, int *admit_slots, int *admit_requests, int *n_admit, int *decode_slots,
                      int *n_decode);
/* The sequence in `slot` sampled a token (is_eos: it was the end-of-sequence id).  *finished = 1 when the sequence
 * ended (EOS, or max_new tokens emitted): its slot and its pages are free for the next plan. */
int blok_batcher_token(blok_batcher_t *batcher, int slot, int is_eos, int *finished);
int blok_batcher_unfinished(const blok_batcher_t *batcher);       /* requests not finished yet (waiting or running) */
int blok_batcher_waiting(const blok_batcher_t *batcher);          /* requests not admitted yet */
long blok_batcher_committed_pages(const blok_batcher_t *batcher); /* pages promised to the running sequences */
int blok_batcher_emitted(const blok_batcher_t *batcher, int request_id); /* tokens emitted for a request */

/* Greedy generation for n_requests prompts at once on a paged model with prefill_chunk >= 1 (HOST arrays): prompt r
 * is prompts[prompt_offsets[r] .. prompt_offsets[r+1]); out holds n_requests * max_new ids, request r's tokens at
 * out + r * max_new, their count in n_out[r].  Each request gets what blok_model_generate gives for it alone (up to
 * the summation order of the batched kernels); the requests share the model's slots and page pool through a
 * blok_batcher: prompts are prefilled as they are admitted, all running sequences step together. */
int blok_model_generate_many(blok_model_t *model, const uint32_t *prompts, const int *prompt_offsets, int n_requests,
                             int max_new, uint32_t *out, int *n_out);

/* Greedy generation for one sequence with HOST token arrays, as generate()
 * (src/kimi_exec.cu:885-890): the prompt is replayed token by token (through
 * blok_model_prefill when prefill_chunk >= 1), then up to max_new tokens are
 * produced, stopping before eos_id.  Returns the count in *n_out. */
int blok_model_generate(blok_model_t *model, const uint32_t *prompt, int n_prompt, int max_new, uint32_t *out,
                        int *n_out);

#ifdef __cplusplus
}
#endif
#endif /* BLOK_B200_H */
