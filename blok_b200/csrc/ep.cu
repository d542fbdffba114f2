// Expert parallelism under the C ABI: a communicator (NCCL for the bootstrap and the small collectives) and the
// expert-parallel form of the batched routed-MoE layer, whose token exchange runs inside this library's own kernels
// over peer memory (NVLink): plain peer stores for the dispatch, plain peer loads for the combine.
//
// The reference runs on one GPU and has no collective at all (src/kimi_exec.cu has no multi-GPU code); per token the
// arithmetic is still the MoE branch of its layer body, :836-877.  Expert e lives on rank e / (experts / world).
//
// One pass on every rank, all on one stream, with NO host synchronisation:
//   1. route the rank's own tokens (router replicated)
//   2. count:    histogram of the assignments by global expert, written into EVERY rank's count table (peer stores),
//                then a flag per peer
//   3. plan:     wait for every rank's row of the table; from the full table each rank derives, without talking,
//                where its rows land in each owner's receive buffer (ordered by expert, then by source rank) and the
//                owner derives the tile table of its grouped GEMM
//   4. dispatch: one CTA per token copies the token's row into the owners' receive buffers (peer stores), the last
//                CTA to finish raises a flag at every peer
//   5. shared expert on the rank's own tokens (needs nothing from the exchange; fills the wait)
//   6. wait for every source's flag, grouped W4A16 GEMM over the receive buffer -> result buffer, flag at every peer
//   7. combine:  wait for every owner's flag; each token reads its eight results from the owners' result buffers
//                (peer loads), weights them in slot order and adds the shared expert (:868-871, :684)
// Flags carry the pass number, so nothing is cleared between passes.  Every wait is bounded and records an error
// word that blok_moe_ep_check returns; indices derived from peers' counts are clamped to the buffers.
//
// No TMA and no multicast touches peer memory: the GEMM reads only this GPU's receive buffer.
#include <dlfcn.h>
#include <nccl.h>

#include <algorithm>
#include <cstring>
#include <mutex>
#include <new>
#include <vector>

#include "common.cuh"
#include "ep_plan.h"
#include "moe_layer.h"
#include "wgemm.h"

namespace blok {

int launch_router_topk(const float *logits, const float *bias, int T, int experts, int topk, float routed_scale,
                       uint16_t *ids, float *wts, int *local_ids, int expert_base, cudaStream_t stream);
int launch_bf16_gemv(const uint16_t *w, const uint16_t *x, uint16_t *y_bf16, float *y_f32, int rows, int cols, int T,
                     cudaStream_t stream);

// ---- NCCL, resolved at run time -------------------------------------------------------------------------------------
// The library is not linked against NCCL: single-GPU users need none, and a process that already holds an NCCL
// (torch's) must not get a second copy.  dlopen by soname returns the copy already loaded, if any.
struct NcclApi {
  void *handle = nullptr;
  ncclResult_t (*GetUniqueId)(ncclUniqueId *) = nullptr;
  ncclResult_t (*CommInitRank)(ncclComm_t *, int, ncclUniqueId, int) = nullptr;
  ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
  ncclResult_t (*CommAbort)(ncclComm_t) = nullptr;
  ncclResult_t (*CommGetAsyncError)(ncclComm_t, ncclResult_t *) = nullptr;
  ncclResult_t (*AllGather)(const void *, void *, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*AllReduce)(const void *, void *, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*Broadcast)(const void *, void *, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t) = nullptr;
  const char *(*GetErrorString)(ncclResult_t) = nullptr;
};

static NcclApi g_nccl;
static std::mutex g_nccl_mu;

static int nccl_load() {
  std::lock_guard<std::mutex> lock(g_nccl_mu);
  if (g_nccl.handle) return BLOK_OK;
  void *h = nullptr;
  const char *override_path = getenv("BLOK_NCCL_LIB");
  const char *names[] = {override_path, "libnccl.so.2", "libnccl.so"};
  for (const char *n : names) {
    if (!n || !*n) continue;
    h = dlopen(n, RTLD_NOW | RTLD_GLOBAL);
    if (h) break;
  }
  if (!h) {
    set_error("blok_comm: libnccl.so.2 not found (%s)", dlerror());
    return BLOK_ERR_COMM;
  }
  NcclApi a;
  a.handle = h;
#define BLOK_NCCL_SYM(field, name)                                      \
  *reinterpret_cast<void **>(&a.field) = dlsym(h, name);                \
  if (!a.field) {                                                       \
    set_error("blok_comm: %s missing from the NCCL library", name);     \
    return BLOK_ERR_COMM;                                               \
  }
  BLOK_NCCL_SYM(GetUniqueId, "ncclGetUniqueId")
  BLOK_NCCL_SYM(CommInitRank, "ncclCommInitRank")
  BLOK_NCCL_SYM(CommDestroy, "ncclCommDestroy")
  BLOK_NCCL_SYM(CommAbort, "ncclCommAbort")
  BLOK_NCCL_SYM(CommGetAsyncError, "ncclCommGetAsyncError")
  BLOK_NCCL_SYM(AllGather, "ncclAllGather")
  BLOK_NCCL_SYM(AllReduce, "ncclAllReduce")
  BLOK_NCCL_SYM(Broadcast, "ncclBroadcast")
  BLOK_NCCL_SYM(GetErrorString, "ncclGetErrorString")
#undef BLOK_NCCL_SYM
  g_nccl = a;
  return BLOK_OK;
}

static int nccl_fail(ncclResult_t r, const char *what) {
  set_error("%s: %s", what, g_nccl.GetErrorString ? g_nccl.GetErrorString(r) : "NCCL error");
  return BLOK_ERR_COMM;
}

#define BLOK_NCCL(call)                                          \
  do {                                                           \
    ncclResult_t r_ = (call);                                    \
    if (r_ != ncclSuccess) return ::blok::nccl_fail(r_, #call);  \
  } while (0)

}  // namespace blok

namespace blok {
struct SymBuf;
}
struct blok_comm {
  ncclComm_t nccl = nullptr;
  int rank = 0, world = 1, device = 0;
  cudaStream_t stream = nullptr;  // set-up collectives
  void *scratch = nullptr;        // world * 128 bytes on the device, for the all-gathers of the set-up
  // the library's own all-reduce for small vectors (the sharded model's one per MoE layer): every rank's receive slots
  // and flags, mapped by every peer
  blok::SymBuf *ar = nullptr;
  unsigned char **ar_peers = nullptr;  // device array: this process's address of every rank's region
  unsigned *ar_state = nullptr;        // device: [0] calls so far, [1] CTAs of the push that are done, [2] error
};

namespace blok {

// A buffer of the same size on every rank, each rank's copy mapped into every other rank's address space.
struct SymBuf {
  void *local = nullptr;
  size_t bytes = 0;
  std::vector<void *> peer;       // peer[r] = this process's address of rank r's copy (peer[rank] = local)
  std::vector<void *> opened;     // bases returned by cudaIpcOpenMemHandle (to close)
};

struct IpcRecord {
  cudaIpcMemHandle_t handle;  // 64 bytes
  unsigned long long offset;  // of the buffer inside the allocation the handle names
  unsigned long long bytes;
  unsigned char pad[128 - sizeof(cudaIpcMemHandle_t) - 16];
};
static_assert(sizeof(IpcRecord) == 128, "IpcRecord must be 128 bytes");

static int sym_alloc(blok_comm *c, size_t bytes, SymBuf *out) {
  out->bytes = (bytes + (2u << 20) - 1) / (2u << 20) * (2u << 20);  // whole 2 MiB blocks: an allocation of its own
  BLOK_CUDA(cudaMalloc(&out->local, out->bytes));
  BLOK_CUDA(cudaMemset(out->local, 0, out->bytes));
  out->peer.assign(c->world, nullptr);
  out->peer[c->rank] = out->local;
  if (c->world == 1) return BLOK_OK;
  IpcRecord mine;
  memset(&mine, 0, sizeof(mine));
  BLOK_CUDA(cudaIpcGetMemHandle(&mine.handle, out->local));
  mine.offset = 0;  // a cudaMalloc of whole 2 MiB blocks is the base of its own allocation
  mine.bytes = out->bytes;
  unsigned char *dev = static_cast<unsigned char *>(c->scratch);
  BLOK_CUDA(cudaMemcpyAsync(dev + (size_t)c->rank * 128, &mine, 128, cudaMemcpyHostToDevice, c->stream));
  BLOK_NCCL(g_nccl.AllGather(dev + (size_t)c->rank * 128, dev, 128, ncclUint8, c->nccl, c->stream));
  std::vector<IpcRecord> all(c->world);
  BLOK_CUDA(cudaMemcpyAsync(all.data(), dev, (size_t)c->world * 128, cudaMemcpyDeviceToHost, c->stream));
  BLOK_CUDA(cudaStreamSynchronize(c->stream));
  for (int r = 0; r < c->world; ++r) {
    if (r == c->rank) continue;
    if (all[r].bytes != out->bytes) {
      set_error("blok_comm: rank %d allocated %llu bytes where rank %d allocated %zu", r, all[r].bytes, c->rank, out->bytes);
      return BLOK_ERR_COMM;
    }
    void *base = nullptr;
    BLOK_CUDA(cudaIpcOpenMemHandle(&base, all[r].handle, cudaIpcMemLazyEnablePeerAccess));
    out->opened.push_back(base);
    out->peer[r] = static_cast<unsigned char *>(base) + all[r].offset;
  }
  return BLOK_OK;
}

static void sym_free(SymBuf *b) {
  for (void *p : b->opened) cudaIpcCloseMemHandle(p);
  b->opened.clear();
  if (b->local) cudaFree(b->local);
  b->local = nullptr;
}

// ---- the library's own all-reduce over peer memory ---------------------------------------------------------------------
// One-shot: every rank stores its vector into its slot of EVERY rank's region (16-byte peer stores over NVLink), then a
// flag that carries the call number; every rank then adds the slots in rank order, so all ranks hold the same bits.
// Two parities of slots: a rank can be one call ahead of a peer that still reads the previous call's slots, never two
// (its own reduce of call n + 1 needs that peer's flag of call n + 1, which the peer stores after its reduce of call n).
// The call number lives on the device, so that a CUDA graph replays the same two launches for every call.
constexpr long kArMaxFloats = 256 * 1024;                 // 1 MB per slot
constexpr size_t kArSlotBytes = (size_t)kArMaxFloats * 4;
constexpr unsigned kArSpinLimit = 1u << 22;

__global__ void __launch_bounds__(256) ar_push_kernel(const float4 *__restrict__ src, long n4, unsigned char *const *__restrict__ peers,
                                                      int world, int rank, unsigned *state) {
  const unsigned call = state[0] + 1u;  // stored back by the last CTA to finish, after every CTA has read it
  const size_t slot = ((size_t)(call & 1u) * world + rank) * kArSlotBytes;
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (long)gridDim.x * blockDim.x) {
    const float4 v = src[i];
    for (int d = 0; d < world; ++d) reinterpret_cast<float4 *>(peers[d] + slot)[i] = v;
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned done = atomicAdd(&state[1], 1u);
    if (done == gridDim.x - 1) {  // every CTA's stores were fenced before its count
      state[1] = 0;
      __threadfence_system();
      for (int d = 0; d < world; ++d) {
        unsigned *flag = reinterpret_cast<unsigned *>(peers[d] + 2 * (size_t)world * kArSlotBytes) + (call & 1u) * world + rank;
        asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(flag), "r"(call) : "memory");
      }
      state[0] = call;
    }
  }
}

__global__ void __launch_bounds__(256) ar_reduce_kernel(float4 *__restrict__ dst, long n4, const unsigned char *__restrict__ local, int world,
                                                        unsigned *state) {
  const unsigned call = state[0];  // this rank's push of the call has finished (stream order)
  const size_t base = (size_t)(call & 1u) * world * kArSlotBytes;
  if ((int)threadIdx.x < world) {
    const unsigned *flag = reinterpret_cast<const unsigned *>(local + 2 * (size_t)world * kArSlotBytes) + (call & 1u) * world + threadIdx.x;
    unsigned it = 0, seen;
    for (;;) {
      asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(flag) : "memory");
      if (seen == call) break;
      if (++it > kArSpinLimit) {  // a peer never signalled: record it and add what is there
        atomicExch(&state[2], 1u + threadIdx.x);
        break;
      }
      __nanosleep(100);
    }
  }
  __syncthreads();
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (long)gridDim.x * blockDim.x) {
    float4 acc = __ldcg(reinterpret_cast<const float4 *>(local + base) + i);  // the peers wrote behind this GPU's L1
    for (int r = 1; r < world; ++r) {
      const float4 v = __ldcg(reinterpret_cast<const float4 *>(local + base + (size_t)r * kArSlotBytes) + i);
      acc.x += v.x;
      acc.y += v.y;
      acc.z += v.z;
      acc.w += v.w;
    }
    dst[i] = acc;
  }
}

// ---- device side ------------------------------------------------------------------------------------------------------
constexpr unsigned kEpSpinLimit = 1u << 22;  // polls (with a 100 ns back-off: about half a second) before a wait gives up

// Layout of a rank's symmetric region.
struct EpRegion {
  size_t table, tflag, dflag, rflag, recv_x, recv_y, total;
};
static EpRegion ep_region(int world, int experts, int hidden, long cap_rows) {
  EpRegion r;
  size_t off = 0;
  auto take = [&](size_t b) { size_t at = off; off = (off + b + 255) / 256 * 256; return at; };
  r.table = take((size_t)world * experts * 4);
  r.tflag = take((size_t)world * 4);
  r.dflag = take((size_t)world * 4);
  r.rflag = take((size_t)world * 4);
  r.recv_x = take((size_t)cap_rows * hidden * 2);
  r.recv_y = take((size_t)cap_rows * hidden * 2);
  r.total = off;
  return r;
}

struct EpParams {
  unsigned char *const *peers;  // [world] this process's address of every rank's region
  int rank, world, experts, per, topk, hidden;
  long cap_rows;
  size_t o_table, o_tflag, o_dflag, o_rflag, o_recv_x, o_recv_y;
  unsigned epoch;
  unsigned *err;     // [1] error word
  int *cursor;       // [experts] next free position among this rank's assignments to an expert
  int *send_base;    // [experts] first row, in the owner's receive buffer, of this rank's assignments to an expert
  int *dst_rank;     // [N] owner of assignment a
  int *dst_row;      // [N] its row in the owner's buffers
  unsigned *done;    // [1] CTAs of the dispatch that have finished
  long long *stats;  // [4] assignments, remote assignments, rows received, tiles
};

__device__ __forceinline__ void st_release_sys(unsigned *p, unsigned v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned *p) {
  unsigned v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
// Waits until *p has reached `epoch` (flags only grow).  Returns false after the poll limit.
__device__ __forceinline__ bool wait_flag(const unsigned *p, unsigned epoch) {
  for (unsigned it = 0; it < kEpSpinLimit; ++it) {
    if ((int)(ld_acquire_sys(p) - epoch) >= 0) return true;
    __nanosleep(100);
  }
  return false;
}

// Step 2.  One CTA: histogram of the rank's N assignments by global expert, into every rank's table row [rank].
__global__ void ep_count_kernel(EpParams p, const uint16_t *__restrict__ ids, int N) {
  extern __shared__ int hist[];
  for (int g = threadIdx.x; g < p.experts; g += blockDim.x) hist[g] = 0;
  __syncthreads();
  for (int a = threadIdx.x; a < N; a += blockDim.x) {
    const int g = ids[a];
    if (g < p.experts) atomicAdd(hist + g, 1);
  }
  __syncthreads();
  for (int g = threadIdx.x; g < p.experts; g += blockDim.x) p.cursor[g] = 0;
  for (int d = 0; d < p.world; ++d) {
    int *row = reinterpret_cast<int *>(p.peers[d] + p.o_table) + (size_t)p.rank * p.experts;
    for (int g = threadIdx.x; g < p.experts; g += blockDim.x) row[g] = hist[g];
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x < p.world)
    st_release_sys(reinterpret_cast<unsigned *>(p.peers[threadIdx.x] + p.o_tflag) + p.rank, p.epoch);
  if (threadIdx.x == 0) {
    int remote = 0;
    for (int g = 0; g < p.experts; ++g)
      if (g / p.per != p.rank) remote += hist[g];
    p.stats[0] = N;
    p.stats[1] = remote;
  }
}

// Step 3.  One CTA (>= experts threads): the full table -> where this rank's rows go, and the owner's tile table.
__global__ void ep_plan_kernel(EpParams p, int *__restrict__ counts, int *__restrict__ offsets, int *__restrict__ tile_expert,
                               int *__restrict__ tile_start, int *__restrict__ tile_count, int *__restrict__ num_tiles,
                               int max_tiles) {
  extern __shared__ int sm[];
  int *tot = sm;                 // [experts] assignments to expert g from all ranks
  int *before = tot + p.experts;  // [experts] of those, from ranks below this one
  int *base = before + p.experts; // [experts] first row of expert g in its owner's buffer
  unsigned char *me = p.peers[p.rank];
  if (threadIdx.x < p.world && !wait_flag(reinterpret_cast<const unsigned *>(me + p.o_tflag) + threadIdx.x, p.epoch))
    atomicExch(p.err, 10u + threadIdx.x);
  __syncthreads();
  const volatile int *table = reinterpret_cast<const volatile int *>(me + p.o_table);
  for (int g = threadIdx.x; g < p.experts; g += blockDim.x) ep_expert_totals(table, p.world, p.experts, p.rank, p.cap_rows, g, tot + g, before + g);
  __syncthreads();
  if (threadIdx.x < p.world) ep_owner_bases(tot, p.per, threadIdx.x, p.cap_rows, base);
  __syncthreads();
  for (int g = threadIdx.x; g < p.experts; g += blockDim.x) p.send_base[g] = base[g] + before[g];
  if (threadIdx.x == 0) {  // this rank as owner: counts, offsets and tiles of 64 rows of one expert
    long rows = 0;
    int overflow = 0;
    const int nt = ep_owner_tiles(tot, p.per, p.rank, p.cap_rows, kWgTileTokens, max_tiles, counts, offsets, tile_expert, tile_start,
                                  tile_count, &rows, &overflow);
    if (overflow) atomicExch(p.err, 20u);
    *num_tiles = nt;
    p.stats[2] = rows;
    p.stats[3] = nt;
  }
}

// Step 4.  One CTA per token: its row goes to the owner of each of its experts; the last CTA raises the flags.
__global__ void ep_dispatch_kernel(EpParams p, const uint16_t *__restrict__ x, const uint16_t *__restrict__ ids, int T) {
  __shared__ int s_rank[16], s_row[16];
  __shared__ bool s_last;
  const int t = blockIdx.x;
  if (t < T) {
    if (threadIdx.x < p.topk) {
      const int a = t * p.topk + threadIdx.x;
      int g = ids[a];
      g = min(g, p.experts - 1);
      const int pos = atomicAdd(p.cursor + g, 1);
      const long row = min((long)p.send_base[g] + pos, p.cap_rows - 1);
      s_rank[threadIdx.x] = g / p.per;
      s_row[threadIdx.x] = (int)row;
      p.dst_rank[a] = g / p.per;
      p.dst_row[a] = (int)row;
    }
    __syncthreads();
    const int units = p.hidden / 8;  // 16-byte pieces of a row
    const uint4 *src = reinterpret_cast<const uint4 *>(x + (size_t)t * p.hidden);
    for (int u = threadIdx.x; u < units; u += blockDim.x) {
      const uint4 v = src[u];
      for (int k = 0; k < p.topk; ++k) {
        uint4 *dst = reinterpret_cast<uint4 *>(p.peers[s_rank[k]] + p.o_recv_x + (size_t)s_row[k] * p.hidden * 2);
        dst[u] = v;
      }
    }
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) s_last = atomicAdd(p.done, 1u) == gridDim.x - 1;
  __syncthreads();
  if (s_last) {
    __threadfence_system();
    if (threadIdx.x < p.world)
      st_release_sys(reinterpret_cast<unsigned *>(p.peers[threadIdx.x] + p.o_dflag) + p.rank, p.epoch);
    if (threadIdx.x == 0) *p.done = 0;
  }
}

// Steps 6 and 7: wait until every rank has raised flag `which` (0: its rows are in my receive buffer; 1: never used
// here) at this rank.
__global__ void ep_wait_kernel(EpParams p, size_t o_flag, unsigned code) {
  if (threadIdx.x < p.world &&
      !wait_flag(reinterpret_cast<const unsigned *>(p.peers[p.rank] + o_flag) + threadIdx.x, p.epoch))
    atomicExch(p.err, code + threadIdx.x);
}

// Step 6, end: this rank's results are complete; tell every rank.
__global__ void ep_signal_kernel(EpParams p, size_t o_flag) {
  __threadfence_system();
  if (threadIdx.x < p.world) st_release_sys(reinterpret_cast<unsigned *>(p.peers[threadIdx.x] + o_flag) + p.rank, p.epoch);
}

// Step 7.  out[t] = bf16(bf16(sum_k w[t,k] * y_k) + shared[t]), y_k read from its owner's result buffer; slot order as
// expert_accum_k / round_bf16_k / add_k (src/kimi_exec.cu:399-407, :248-251).
__global__ void ep_combine_kernel(EpParams p, const float *__restrict__ wts, const uint16_t *__restrict__ shared, int T,
                                  uint16_t *__restrict__ out) {
  __shared__ int s_rank[16], s_row[16];
  __shared__ float s_w[16];
  const int t = blockIdx.x;
  if (threadIdx.x < p.world &&
      !wait_flag(reinterpret_cast<const unsigned *>(p.peers[p.rank] + p.o_rflag) + threadIdx.x, p.epoch))
    atomicExch(p.err, 40u + threadIdx.x);
  if (threadIdx.x < p.topk) {
    const int a = t * p.topk + threadIdx.x;
    s_rank[threadIdx.x] = p.dst_rank[a];
    s_row[threadIdx.x] = p.dst_row[a];
    s_w[threadIdx.x] = wts[a];
  }
  __syncthreads();
  const int units = p.hidden / 8;
  for (int u = threadIdx.x; u < units; u += blockDim.x) {
    float o[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int k = 0; k < p.topk; ++k) {
      const uint4 *src = reinterpret_cast<const uint4 *>(p.peers[s_rank[k]] + p.o_recv_y + (size_t)s_row[k] * p.hidden * 2);
      const uint4 v = __ldcg(src + u);
      const float w = s_w[k];
      o[0] = fmaf(bf16lo(v.x), w, o[0]); o[1] = fmaf(bf16hi(v.x), w, o[1]);
      o[2] = fmaf(bf16lo(v.y), w, o[2]); o[3] = fmaf(bf16hi(v.y), w, o[3]);
      o[4] = fmaf(bf16lo(v.z), w, o[4]); o[5] = fmaf(bf16hi(v.z), w, o[5]);
      o[6] = fmaf(bf16lo(v.w), w, o[6]); o[7] = fmaf(bf16hi(v.w), w, o[7]);
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) o[i] = round_bf16(o[i]);
    if (shared) {
      const uint4 s = reinterpret_cast<const uint4 *>(shared + (size_t)t * p.hidden)[u];
      o[0] = round_bf16(o[0] + bf16lo(s.x)); o[1] = round_bf16(o[1] + bf16hi(s.x));
      o[2] = round_bf16(o[2] + bf16lo(s.y)); o[3] = round_bf16(o[3] + bf16hi(s.y));
      o[4] = round_bf16(o[4] + bf16lo(s.z)); o[5] = round_bf16(o[5] + bf16hi(s.z));
      o[6] = round_bf16(o[6] + bf16lo(s.w)); o[7] = round_bf16(o[7] + bf16hi(s.w));
    }
    uint4 r;
    r.x = pack_bf16x2(o[0], o[1]); r.y = pack_bf16x2(o[2], o[3]); r.z = pack_bf16x2(o[4], o[5]); r.w = pack_bf16x2(o[6], o[7]);
    reinterpret_cast<uint4 *>(out + (size_t)t * p.hidden)[u] = r;
  }
}

}  // namespace blok

using namespace blok;

struct blok_moe_ep {
  blok_comm *comm = nullptr;
  blok_moe_layer *layer = nullptr;  // this rank's shard: workspace of the router, the shared expert and the grouped GEMM
  blok_moe_weights w;
  int max_tokens = 0;
  long cap_rows = 0;
  SymBuf sym;
  EpRegion reg;
  unsigned char **d_peers = nullptr;  // device copy of sym.peer
  void *dws = nullptr;                // cursor, send_base, dst_rank, dst_row, done, err, stats
  int *cursor = nullptr, *send_base = nullptr, *dst_rank = nullptr, *dst_row = nullptr;
  unsigned *done = nullptr, *err = nullptr;
  long long *stats = nullptr;
  unsigned epoch = 0;
  bool profile = false;          // record an event between the phases of a pass
  cudaEvent_t ev[7] = {};
};

// ---- communicator -------------------------------------------------------------------------------------------------------
extern "C" int blok_comm_unique_id(void *id_out) {
  BLOK_REQUIRE(id_out, BLOK_ERR_ARG, "blok_comm_unique_id: null pointer");
  if (int rc = nccl_load()) return rc;
  static_assert(sizeof(ncclUniqueId) == BLOK_COMM_ID_BYTES, "ncclUniqueId is 128 bytes");
  ncclUniqueId id;
  BLOK_NCCL(g_nccl.GetUniqueId(&id));
  memcpy(id_out, &id, sizeof(id));
  return BLOK_OK;
}

extern "C" int blok_comm_create(const void *unique_id, int rank, int world, blok_comm_t **out) {
  BLOK_REQUIRE(out, BLOK_ERR_ARG, "blok_comm_create: null pointer");
  BLOK_REQUIRE(world >= 1 && world <= 64 && rank >= 0 && rank < world, BLOK_ERR_ARG, "blok_comm_create: rank %d of %d", rank,
               world);
  BLOK_REQUIRE(world == 1 || unique_id, BLOK_ERR_ARG, "blok_comm_create: unique_id missing");
  blok_comm *c = new (std::nothrow) blok_comm();
  BLOK_REQUIRE(c, BLOK_ERR_ARG, "blok_comm_create: out of host memory");
  c->rank = rank;
  c->world = world;
  auto fail = [&](int rc) {
    blok_comm_destroy(c);
    return rc;
  };
  cudaError_t e = cudaGetDevice(&c->device);
  if (e != cudaSuccess) return fail(cuda_fail(e, "cudaGetDevice"));
  if ((e = cudaStreamCreateWithFlags(&c->stream, cudaStreamNonBlocking)) != cudaSuccess) return fail(cuda_fail(e, "cudaStreamCreate"));
  if ((e = cudaMalloc(&c->scratch, (size_t)world * 128)) != cudaSuccess) return fail(cuda_fail(e, "cudaMalloc(comm scratch)"));
  if (world > 1) {
    if (int rc = nccl_load()) return fail(rc);
    ncclUniqueId id;
    memcpy(&id, unique_id, sizeof(id));
    ncclResult_t r = g_nccl.CommInitRank(&c->nccl, world, id, rank);
    if (r != ncclSuccess) return fail(nccl_fail(r, "ncclCommInitRank"));
    // the regions of the library's own all-reduce: 2 parities x world slots, then 2 x world flags
    c->ar = new (std::nothrow) SymBuf();
    if (!c->ar) return fail(BLOK_ERR_ARG);
    if (int rc = sym_alloc(c, 2 * (size_t)world * kArSlotBytes + 4096, c->ar)) return fail(rc);
    if ((e = cudaMalloc(&c->ar_peers, (size_t)world * sizeof(void *))) != cudaSuccess) return fail(cuda_fail(e, "cudaMalloc(all-reduce peers)"));
    if ((e = cudaMemcpy(c->ar_peers, c->ar->peer.data(), (size_t)world * sizeof(void *), cudaMemcpyHostToDevice)) != cudaSuccess)
      return fail(cuda_fail(e, "cudaMemcpy(all-reduce peers)"));
    if ((e = cudaMalloc(&c->ar_state, 64)) != cudaSuccess) return fail(cuda_fail(e, "cudaMalloc(all-reduce state)"));
    if ((e = cudaMemset(c->ar_state, 0, 64)) != cudaSuccess) return fail(cuda_fail(e, "cudaMemset(all-reduce state)"));
    // nobody stores into a peer's region before every rank has mapped and cleared its own
    if ((e = cudaMemsetAsync(c->scratch, 0, 128, c->stream)) != cudaSuccess) return fail(cuda_fail(e, "cudaMemsetAsync"));
    r = g_nccl.AllReduce(c->scratch, c->scratch, 1, ncclFloat32, ncclSum, c->nccl, c->stream);
    if (r != ncclSuccess) return fail(nccl_fail(r, "ncclAllReduce(set-up barrier)"));
    if ((e = cudaStreamSynchronize(c->stream)) != cudaSuccess) return fail(cuda_fail(e, "cudaStreamSynchronize"));
  }
  *out = c;
  return BLOK_OK;
}

extern "C" int blok_comm_destroy(blok_comm_t *c) {
  if (!c) return BLOK_OK;
  if (c->ar) {
    sym_free(c->ar);
    delete c->ar;
  }
  if (c->ar_peers) cudaFree(c->ar_peers);
  if (c->ar_state) cudaFree(c->ar_state);
  if (c->nccl) g_nccl.CommDestroy(c->nccl);
  if (c->scratch) cudaFree(c->scratch);
  if (c->stream) cudaStreamDestroy(c->stream);
  delete c;
  return BLOK_OK;
}

extern "C" int blok_comm_rank(const blok_comm_t *c) { return c ? c->rank : -1; }
extern "C" int blok_comm_world(const blok_comm_t *c) { return c ? c->world : 0; }

extern "C" int blok_comm_check(blok_comm_t *c) {
  BLOK_REQUIRE(c, BLOK_ERR_ARG, "blok_comm_check: null pointer");
  if (!c->nccl) return BLOK_OK;
  if (c->ar_state) {  // the caller has synchronised the streams it used; a peer that never signalled left its rank + 1 here
    unsigned err = 0;
    BLOK_CUDA(cudaMemcpy(&err, c->ar_state + 2, sizeof(err), cudaMemcpyDeviceToHost));
    if (err) {
      BLOK_CUDA(cudaMemset(c->ar_state + 2, 0, sizeof(err)));
      set_error("blok_comm_all_reduce_f32: rank %u never signalled its part of an all-reduce", err - 1);
      return BLOK_ERR_TIMEOUT;
    }
  }
  ncclResult_t st = ncclSuccess;
  BLOK_NCCL(g_nccl.CommGetAsyncError(c->nccl, &st));
  if (st != ncclSuccess && st != ncclInProgress) return nccl_fail(st, "blok_comm_check: asynchronous NCCL error");
  return BLOK_OK;
}

extern "C" int blok_comm_all_reduce_f32(blok_comm_t *c, float *buf, long n, blok_stream_t stream) {
  BLOK_REQUIRE(c && (buf || n == 0) && n >= 0, BLOK_ERR_ARG, "blok_comm_all_reduce_f32: bad argument");
  if (c->world == 1 || n == 0) return BLOK_OK;
  // up to 1 MB: the library's own kernels over peer memory (two launches, no library call; the same bits on every
  // rank); BLOK_COMM_ALLREDUCE=nccl in the environment, longer or unaligned vectors: ncclAllReduce
  const char *how = getenv("BLOK_COMM_ALLREDUCE");
  if (c->ar && n <= kArMaxFloats && n % 4 == 0 && (reinterpret_cast<uintptr_t>(buf) & 15) == 0 && !(how && strcmp(how, "nccl") == 0)) {
    const long n4 = n / 4;
    const int ctas = (int)std::min<long>(64, (n4 + 255) / 256);
    ar_push_kernel<<<ctas, 256, 0, (cudaStream_t)stream>>>(reinterpret_cast<const float4 *>(buf), n4, c->ar_peers, c->world, c->rank,
                                                         c->ar_state);
    if (int rc = launch_status("ar_push_kernel")) return rc;
    ar_reduce_kernel<<<(int)std::min<long>(148, (n4 + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
        reinterpret_cast<float4 *>(buf), n4, static_cast<const unsigned char *>(c->ar->local), c->world, c->ar_state);
    return launch_status("ar_reduce_kernel");
  }
  BLOK_NCCL(g_nccl.AllReduce(buf, buf, (size_t)n, ncclFloat32, ncclSum, c->nccl, (cudaStream_t)stream));
  return BLOK_OK;
}

extern "C" int blok_comm_broadcast(blok_comm_t *c, void *buf, long bytes, int root, blok_stream_t stream) {
  BLOK_REQUIRE(c && (buf || bytes == 0) && bytes >= 0 && root >= 0 && root < c->world, BLOK_ERR_ARG,
               "blok_comm_broadcast: bad argument");
  if (c->world == 1 || bytes == 0) return BLOK_OK;
  BLOK_NCCL(g_nccl.Broadcast(buf, buf, (size_t)bytes, ncclUint8, root, c->nccl, (cudaStream_t)stream));
  return BLOK_OK;
}

// The plan of one rank from the gathered count table, on the HOST: the same functions the plan kernel runs.
extern "C" int blok_ep_plan_host(const int *table, int world, int experts, int rank, long cap_rows, int max_tiles, int *send_base,
                                 int *counts, int *offsets, int *tile_expert, int *tile_start, int *tile_count, int *num_tiles) {
  BLOK_REQUIRE(table && send_base && counts && offsets && tile_expert && tile_start && tile_count && num_tiles, BLOK_ERR_ARG,
               "blok_ep_plan_host: null pointer");
  BLOK_REQUIRE(world >= 1 && experts >= world && experts % world == 0 && rank >= 0 && rank < world && cap_rows >= 0 && max_tiles >= 0,
               BLOK_ERR_SHAPE, "blok_ep_plan_host: rank %d of %d, %d experts", rank, world, experts);
  const int per = experts / world;
  std::vector<int> tot(experts), before(experts), base(experts);
  for (int g = 0; g < experts; ++g) ep_expert_totals(table, world, experts, rank, cap_rows, g, &tot[g], &before[g]);
  for (int d = 0; d < world; ++d) ep_owner_bases(tot.data(), per, d, cap_rows, base.data());
  for (int g = 0; g < experts; ++g) send_base[g] = base[g] + before[g];
  long rows = 0;
  int overflow = 0;
  *num_tiles = ep_owner_tiles(tot.data(), per, rank, cap_rows, kWgTileTokens, max_tiles, counts, offsets, tile_expert, tile_start,
                              tile_count, &rows, &overflow);
  if (overflow) {
    set_error("blok_ep_plan_host: rank %d would receive more than %ld rows", rank, cap_rows);
    return BLOK_ERR_ROUTE;
  }
  return BLOK_OK;
}

// ---- expert-parallel layer ------------------------------------------------------------------------------------------------
extern "C" int blok_moe_ep_destroy(blok_moe_ep_t *ep) {
  if (!ep) return BLOK_OK;
  cudaDeviceSynchronize();
  if (ep->layer) blok_moe_layer_destroy(ep->layer);
  for (cudaEvent_t e : ep->ev)
    if (e) cudaEventDestroy(e);
  sym_free(&ep->sym);
  if (ep->d_peers) cudaFree(ep->d_peers);
  if (ep->dws) cudaFree(ep->dws);
  delete ep;
  return BLOK_OK;
}

extern "C" int blok_moe_ep_create(blok_comm_t *comm, const blok_moe_weights *w, int max_tokens, blok_moe_ep_t **out) {
  BLOK_REQUIRE(comm && w && out, BLOK_ERR_ARG, "blok_moe_ep_create: null pointer");
  BLOK_REQUIRE(max_tokens >= 1, BLOK_ERR_ARG, "blok_moe_ep_create: max_tokens must be >= 1");
  BLOK_REQUIRE(w->experts % comm->world == 0, BLOK_ERR_SHAPE, "blok_moe_ep_create: %d experts do not divide over %d ranks",
               w->experts, comm->world);
  const int per = w->experts / comm->world;
  BLOK_REQUIRE(w->experts_local == per && w->expert_base == comm->rank * per, BLOK_ERR_SHAPE,
               "blok_moe_ep_create: rank %d must hold experts [%d, %d), the weights describe [%d, %d)", comm->rank,
               comm->rank * per, (comm->rank + 1) * per, w->expert_base, w->expert_base + w->experts_local);
  BLOK_REQUIRE(w->hidden % 512 == 0 && w->inter % 512 == 0 && w->topk <= 16 && w->experts <= 1024 &&
                   (w->shared_inter == 0 || w->shared_inter % 512 == 0),
               BLOK_ERR_SHAPE, "blok_moe_ep_create: hidden/inter/shared_inter must be multiples of 512, topk <= 16");
  const long cap = (long)comm->world * max_tokens * w->topk;  // every assignment of every rank could land here
  BLOK_REQUIRE(cap < (1L << 30), BLOK_ERR_SHAPE, "blok_moe_ep_create: capacity of %ld rows is too large", cap);
  blok_moe_ep *ep = new (std::nothrow) blok_moe_ep();
  BLOK_REQUIRE(ep, BLOK_ERR_ARG, "blok_moe_ep_create: out of host memory");
  ep->comm = comm;
  ep->w = *w;
  ep->max_tokens = max_tokens;
  ep->cap_rows = cap;
  auto fail = [&](int rc) {
    blok_moe_ep_destroy(ep);
    return rc;
  };
  // the inner handle sizes the grouped GEMM's scratch for `cap` assignments and the router / shared expert for the
  // rank's own tokens (its token capacity covers both)
  if (int rc = blok_moe_layer_create(w, (int)std::max<long>(2, (long)comm->world * max_tokens), &ep->layer)) return fail(rc);
  ep->reg = ep_region(comm->world, w->experts, w->hidden, cap);
  if (int rc = sym_alloc(comm, ep->reg.total, &ep->sym)) return fail(rc);
  cudaError_t e = cudaMalloc(&ep->d_peers, (size_t)comm->world * sizeof(void *));
  if (e != cudaSuccess) return fail(cuda_fail(e, "cudaMalloc(peer table)"));
  e = cudaMemcpy(ep->d_peers, ep->sym.peer.data(), (size_t)comm->world * sizeof(void *), cudaMemcpyHostToDevice);
  if (e != cudaSuccess) return fail(cuda_fail(e, "cudaMemcpy(peer table)"));
  const size_t N = (size_t)max_tokens * w->topk;
  size_t off = 0;
  auto take = [&](size_t b) { size_t at = off; off = (off + b + 255) / 256 * 256; return at; };
  const size_t o_cur = take((size_t)w->experts * 4), o_sb = take((size_t)w->experts * 4), o_dr = take(N * 4), o_dw = take(N * 4);
  const size_t o_done = take(4), o_err = take(4), o_stats = take(4 * 8);
  if ((e = cudaMalloc(&ep->dws, off)) != cudaSuccess) return fail(cuda_fail(e, "cudaMalloc(ep workspace)"));
  if ((e = cudaMemset(ep->dws, 0, off)) != cudaSuccess) return fail(cuda_fail(e, "cudaMemset(ep workspace)"));
  unsigned char *b = static_cast<unsigned char *>(ep->dws);
  ep->cursor = (int *)(b + o_cur); ep->send_base = (int *)(b + o_sb); ep->dst_rank = (int *)(b + o_dr); ep->dst_row = (int *)(b + o_dw);
  ep->done = (unsigned *)(b + o_done); ep->err = (unsigned *)(b + o_err); ep->stats = (long long *)(b + o_stats);
  if ((e = cudaDeviceSynchronize()) != cudaSuccess) return fail(cuda_fail(e, "cudaDeviceSynchronize"));
  *out = ep;
  return BLOK_OK;
}

extern "C" int blok_moe_ep_forward(blok_moe_ep_t *ep, const blok_bf16_t *x, int T, blok_bf16_t *y, uint16_t *ids_out,
                                   float *wts_out, blok_stream_t stream_) {
  BLOK_REQUIRE(ep, BLOK_ERR_ARG, "blok_moe_ep_forward: null handle");
  BLOK_REQUIRE(T >= 0 && T <= ep->max_tokens, BLOK_ERR_SHAPE, "blok_moe_ep_forward: T=%d exceeds max_tokens %d", T, ep->max_tokens);
  BLOK_REQUIRE(T == 0 || (x && y), BLOK_ERR_ARG, "blok_moe_ep_forward: null pointer");
  cudaStream_t stream = (cudaStream_t)stream_;
  blok_moe_layer *L = ep->layer;
  const blok_moe_weights &w = ep->w;
  const int N = T * w.topk;
  int rc;
  EpParams p;
  p.peers = ep->d_peers;
  p.rank = ep->comm->rank; p.world = ep->comm->world; p.experts = w.experts; p.per = w.experts / p.world; p.topk = w.topk;
  p.hidden = w.hidden; p.cap_rows = ep->cap_rows;
  p.o_table = ep->reg.table; p.o_tflag = ep->reg.tflag; p.o_dflag = ep->reg.dflag; p.o_rflag = ep->reg.rflag;
  p.o_recv_x = ep->reg.recv_x; p.o_recv_y = ep->reg.recv_y;
  p.epoch = ++ep->epoch;
  p.err = ep->err; p.cursor = ep->cursor; p.send_base = ep->send_base; p.dst_rank = ep->dst_rank; p.dst_row = ep->dst_row;
  p.done = ep->done; p.stats = ep->stats;

  auto mark = [&](int i) {
    if (ep->profile) cudaEventRecord(ep->ev[i], stream);
  };
  mark(0);
  // 1. route this rank's tokens (fp32 logits, unrounded, :297; then the top-k kernel)
  if (T > 0) {
    if (w.experts % 128 == 0) {  // the same kernel as blok_moe_batched at every T, so that the two agree bit for bit
      const int tt = (T + kWgTileTokens - 1) / kWgTileTokens;
      if ((rc = launch_identity_tiles(T, L->b_ttile_expert, L->b_ttile_start, L->b_ttile_count, L->b_num_ttiles, stream))) return rc;
      WgArgs r;
      r.w_a = w.router_w; r.w_b = nullptr; r.s_a = r.s_b = nullptr; r.expert_stride_rows = 0; r.x = x; r.x_index = nullptr;
      r.K = w.hidden; r.R = w.experts; r.out_bf16 = nullptr; r.out_f32 = L->logits;
      r.tile_expert = L->b_ttile_expert; r.tile_start = L->b_ttile_start; r.tile_count = L->b_ttile_count;
      r.num_tiles = L->b_num_ttiles; r.out_index = nullptr; r.n_rows = T; r.identity_tiles = 1;
      r.splitk_ws = L->b_splitk; r.splitk_bytes = L->b_splitk_bytes;
      if ((rc = launch_wgemm(WG_BF16_PLAIN, r, tt, stream))) return rc;
    } else {
      for (int t0 = 0; t0 < T; t0 += 8)
        if ((rc = launch_bf16_gemv(w.router_w, x + (size_t)t0 * w.hidden, nullptr, L->logits + (size_t)t0 * w.experts, w.experts,
                                   w.hidden, std::min(8, T - t0), stream)))
          return rc;
    }
    if ((rc = launch_router_topk(L->logits, w.router_bias, T, w.experts, w.topk, w.routed_scale, L->ids, L->wts, nullptr, 0, stream)))
      return rc;
  }
  mark(1);
  // 2-4. counts to every rank, plan, rows to their owners
  ep_count_kernel<<<1, 1024, (size_t)w.experts * sizeof(int), stream>>>(p, L->ids, N);
  if ((rc = launch_status("ep_count_kernel"))) return rc;
  const int max_tiles = (int)std::min<long>(L->b_max_tiles, (ep->cap_rows + kWgTileTokens - 1) / kWgTileTokens + p.per);
  ep_plan_kernel<<<1, 512, (size_t)3 * w.experts * sizeof(int), stream>>>(p, L->b_counts, L->b_offsets, L->b_tile_expert,
                                                                        L->b_tile_start, L->b_tile_count, L->b_num_tiles, max_tiles);
  if ((rc = launch_status("ep_plan_kernel"))) return rc;
  ep_dispatch_kernel<<<std::max(T, 1), 256, 0, stream>>>(p, x, L->ids, T);
  if ((rc = launch_status("ep_dispatch_kernel"))) return rc;
  mark(2);
  // 5. the shared expert on the rank's own tokens while the rows travel
  const uint16_t *shared = nullptr;
  if (w.shared_inter > 0 && T > 0) {
    if ((rc = blok_moe_shared(L, x, T, L->b_sout, stream_))) return rc;
    shared = L->b_sout;
  }
  mark(3);
  // 6. every source's rows are here -> grouped GEMM over the receive buffer -> tell every rank
  ep_wait_kernel<<<1, 64, 0, stream>>>(p, ep->reg.dflag, 30u);
  if ((rc = launch_status("ep_wait_kernel"))) return rc;
  mark(4);
  {
    unsigned char *me = static_cast<unsigned char *>(ep->sym.local);
    const uint16_t *rx = reinterpret_cast<const uint16_t *>(me + ep->reg.recv_x);
    uint16_t *ry = reinterpret_cast<uint16_t *>(me + ep->reg.recv_y);
    WgArgs g;
    g.w_a = w.gate_w; g.w_b = w.up_w; g.s_a = w.gate_s; g.s_b = w.up_s; g.expert_stride_rows = w.inter;
    g.x = rx; g.x_index = nullptr; g.K = w.hidden; g.R = w.inter; g.out_bf16 = L->b_mid; g.out_f32 = nullptr;
    g.tile_expert = L->b_tile_expert; g.tile_start = L->b_tile_start; g.tile_count = L->b_tile_count;
    g.num_tiles = L->b_num_tiles; g.out_index = nullptr; g.small_limit = L->b_num_tiles + 1;
    g.n_rows = (int)std::min<long>(ep->cap_rows, (long)std::max(N, 1) );  // what a balanced routing sends here; picks the kernel
    if ((rc = launch_wgemm(WG_I4_SWIGLU, g, max_tiles, stream))) return rc;
    WgArgs d = g;
    d.w_a = w.down_w; d.w_b = nullptr; d.s_a = w.down_s; d.s_b = nullptr; d.expert_stride_rows = w.hidden;
    d.x = L->b_mid; d.K = w.inter; d.R = w.hidden; d.out_bf16 = ry;
    if ((rc = launch_wgemm(WG_I4_PLAIN, d, max_tiles, stream))) return rc;
  }
  mark(5);
  ep_signal_kernel<<<1, 64, 0, stream>>>(p, ep->reg.rflag);
  if ((rc = launch_status("ep_signal_kernel"))) return rc;
  // 7. combine (waits for every owner's flag)
  if (T > 0) {
    ep_combine_kernel<<<T, 256, 0, stream>>>(p, L->wts, shared, T, y);
    if ((rc = launch_status("ep_combine_kernel"))) return rc;
    if (ids_out) BLOK_CUDA(cudaMemcpyAsync(ids_out, L->ids, (size_t)N * sizeof(uint16_t), cudaMemcpyDeviceToDevice, stream));
    if (wts_out) BLOK_CUDA(cudaMemcpyAsync(wts_out, L->wts, (size_t)N * sizeof(float), cudaMemcpyDeviceToDevice, stream));
  } else {
    // a rank without tokens still has to see the owners' flags of this pass before the next pass reuses the buffers
    ep_wait_kernel<<<1, 64, 0, stream>>>(p, ep->reg.rflag, 40u);
    if ((rc = launch_status("ep_wait_kernel"))) return rc;
  }
  mark(6);
  return BLOK_OK;
}

extern "C" int blok_moe_ep_profile(blok_moe_ep_t *ep, int on) {
  BLOK_REQUIRE(ep, BLOK_ERR_ARG, "blok_moe_ep_profile: null handle");
  if (on)
    for (cudaEvent_t &e : ep->ev)
      if (!e) BLOK_CUDA(cudaEventCreate(&e));
  ep->profile = on != 0;
  return BLOK_OK;
}

extern "C" int blok_moe_ep_phase_ms(blok_moe_ep_t *ep, float *host_out6) {
  BLOK_REQUIRE(ep && host_out6, BLOK_ERR_ARG, "blok_moe_ep_phase_ms: null pointer");
  BLOK_REQUIRE(ep->profile && ep->ev[6], BLOK_ERR_STATE, "blok_moe_ep_phase_ms: profiling is off");
  BLOK_CUDA(cudaEventSynchronize(ep->ev[6]));
  for (int i = 0; i < 6; ++i) BLOK_CUDA(cudaEventElapsedTime(host_out6 + i, ep->ev[i], ep->ev[i + 1]));
  return BLOK_OK;
}

extern "C" int blok_moe_ep_check(blok_moe_ep_t *ep, blok_stream_t stream) {
  BLOK_REQUIRE(ep, BLOK_ERR_ARG, "blok_moe_ep_check: null handle");
  BLOK_CUDA(cudaStreamSynchronize((cudaStream_t)stream));
  unsigned err = 0;
  BLOK_CUDA(cudaMemcpy(&err, ep->err, sizeof(err), cudaMemcpyDeviceToHost));
  if (err) {
    BLOK_CUDA(cudaMemset(ep->err, 0, sizeof(err)));
    BLOK_CUDA(cudaMemset(ep->done, 0, sizeof(unsigned)));
    set_error("blok_moe_ep_forward: device-side wait %u gave up (10+r: counts of rank r, 20: receive buffer full, 30+r: rows of "
              "rank r, 40+r: results of rank r)", err);
    return err == 20u ? BLOK_ERR_ROUTE : BLOK_ERR_TIMEOUT;
  }
  if (int rc = blok_moe_layer_check(ep->layer, stream)) return rc;
  return blok_comm_check(ep->comm);
}

extern "C" int blok_moe_ep_stats(blok_moe_ep_t *ep, long long *host_out4, blok_stream_t stream) {
  BLOK_REQUIRE(ep && host_out4, BLOK_ERR_ARG, "blok_moe_ep_stats: null pointer");
  BLOK_CUDA(cudaStreamSynchronize((cudaStream_t)stream));
  BLOK_CUDA(cudaMemcpy(host_out4, ep->stats, 4 * sizeof(long long), cudaMemcpyDeviceToHost));
  return BLOK_OK;
}
