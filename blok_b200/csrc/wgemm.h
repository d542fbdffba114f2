// Interface of the weight-streaming GEMM (wgemm.cu).
#pragma once
#include <cuda_runtime.h>
#include <cstddef>
#include <cstdint>

namespace blok {

enum { WG_BF16_PLAIN = 0, WG_BF16_SWIGLU = 1, WG_I4_SWIGLU = 2, WG_I4_PLAIN = 3 };
constexpr int kWgTileTokens = 64;
constexpr int kWgStreamTokens = 64;  // bf16 weights over up to this many rows take the weight-streaming kernel (wgemm_stream.cu)
constexpr int kWgSmallTokens = 8;  // groups of up to this many tokens take the mat-vec-style kernel (wgemv_small.cu: four per pass)

struct WgArgs {
  const void *w_a;
  const void *w_b;
  const uint16_t *s_a;
  const uint16_t *s_b;
  long expert_stride_rows;
  const uint16_t *x;
  const int *x_index;
  int K;
  int R;
  uint16_t *out_bf16;
  float *out_f32;
  const int *tile_expert;
  const int *tile_start;
  const int *tile_count;
  const int *num_tiles;
  const int *out_index;
  int identity_tiles = 0;  // the tiles are consecutive 64-row blocks of x (one group: a dense layer over n_rows tokens)
  int n_rows = 0;  // rows of x the launch covers (tokens, or token-expert assignments): picks the kernel
  int small_max = 0;  // > 0: tiles of at most this many tokens are somebody else's (wgemv_small.cu) and are skipped
  // INT4 modes, optional: a device word in which the small-group kernel leaves the group size up to which it took the
  // launch's tiles (it takes every group when the larger ones are few); the GEMM kernel behind it skips those
  int *small_limit = nullptr;
  // bf16 modes over identity tiles: scratch for the K-split partial sums, see wgemm_splitk_bytes; NULL: no split
  float *splitk_ws = nullptr;
  size_t splitk_bytes = 0;
};

// Picks the kernels of a launch.  INT4 modes: the small-group kernel first (wgemv_small.cu), then for what it left the
// tcgen05 kernel (wgemm_tc.cu) from 256 assignments on, below that the mma.sync kernel.  bf16 modes: up to
// kWgStreamTokens rows of a dense product the weight-streaming kernel (wgemm_stream.cu); from 640 tokens on the tcgen05
// kernel; in between, and for shapes the others do not cover, the mma.sync kernel with its K-split.
// BLOK_WGEMM_IMPL=mma / =tc in the environment forces one GEMM kernel for every row (no small-group or streaming kernel).
int launch_wgemm(int mode, const WgArgs &args, int max_tiles, cudaStream_t stream);

// A bf16 product over few tiles of tokens has (R / 128 or R / 64) x tiles CTAs, far fewer than the GPU has SMs (3 per
// tile for a 384-expert router): the mma.sync kernel then splits K over blockIdx.z so that about two CTAs per SM run,
// writes fp32 partial sums to args.splitk_ws and a second kernel adds them in split order and applies the epilogue.
// The factor depends on the launch's shape (mode, K, R, number of token tiles), so two launches of the same shape give
// the same bits.  wgemm_splitk_bytes: the scratch that serves every launch of up to max_rows rows.
int wgemm_splitk_factor(int mode, int K, int R, int tiles);
size_t wgemm_splitk_bytes(int mode, int K, int R, int max_rows);

// Fills the tile arrays with consecutive 64-row tiles of T rows (one group, expert 0): a dense layer.
int launch_identity_tiles(int T, int *tile_expert, int *tile_start, int *tile_count, int *num_tiles, cudaStream_t stream);

// The INT4 modes for groups of up to kWgSmallTokens tokens (every group when the larger ones are few, see
// WgArgs::small_limit): streams the weights like the batch-1 decode kernel and leaves the other groups alone.  launch_wgemm runs it in front of the kernel that takes the rest
// (BLOK_WGEMM_SMALL=0 in the environment: every group through the GEMM kernels).
bool wgemv_small_supports(int mode, const WgArgs &args, int max_tiles);
int launch_wgemv_small(int mode, const WgArgs &args, cudaStream_t stream);

// The bf16 modes over 1..kWgStreamTokens rows of x (identity tiles): every warp streams its 16 weight rows through a
// cp.async ring, the activations are double buffered (wgemm_stream.cu).  *splits > 1: K was split and the partial sums
// wait in args.splitk_ws for wgemm_splitk_reduce_kernel (launch_wgemm runs it).  wgemm_stream_split: the split of a shape.
bool wgemm_stream_supports(int mode, const WgArgs &args);
int wgemm_stream_split(int mode, int K, int R);
int launch_wgemm_stream(int mode, const WgArgs &args, int *splits, cudaStream_t stream);
// One dense product through launch_wgemm without tile tables: out[T, R] = W[R, K] x[T, K] (mode WG_BF16_PLAIN; bf16 or
// fp32 output) or the SwiGLU front half of (w_a = gate, w_b = up) (mode WG_BF16_SWIGLU), for 1 <= T <= kWgStreamTokens.
int launch_wgemm_rows(int mode, const void *w_a, const void *w_b, const uint16_t *x, uint16_t *out_bf16, float *out_f32, int R, int K,
                      int T, float *splitk_ws, size_t splitk_bytes, cudaStream_t stream);

bool wgemm_tc_supports(int mode, const WgArgs &args);
int launch_wgemm_tc(int mode, const WgArgs &args, int max_tiles, cudaStream_t stream);
// *out becomes non-zero if a tcgen05 GEMM CTA has given up on a barrier since the last call (the flag is cleared).
int wgemm_tc_take_error(unsigned *out);

}  // namespace blok
