// bf16 mat-vec for up to 8 tokens on mma.sync tensor cores, the dense SwiGLU MLP,
// RMSNorm and the rounded residual add.
// Reference arithmetic: src/kimi_exec.cu:272-298 (matvec_bf16_k, matvec_bf16_f32_k),
// :674-686 (bf16_mlp), :258-270 (rmsnorm_k), :248-251 (add_k).
//
// Mapping of the mat-vec: a warp owns 16 weight rows (lane group g = lane/4 owns
// rows g and g+8); a k-step is 32 columns, lane t = lane%4 loads the 8 consecutive
// bf16 (one uint4) at column 8t of each of its two rows.  The B operand's column n
// is token n, so lane (g, t) reads the same 8 columns of token g's activation row
// from shared memory.  D[row][token] accumulates in fp32.
#include <algorithm>

#include "bf16_mma.cuh"
#include "wgemm.h"

namespace blok {

// mode 0: y[t, row] plain mat-vec (rows from w_a only; CTA = 16 rows).
// mode 1: SwiGLU front half (CTA = 8 gate rows from w_a + the same 8 up rows
//         from w_b); writes mid = bf16(bf16(silu(bf16 g)) * bf16 u) to y_bf16 [T, rows].
template <int MODE>
__global__ void __launch_bounds__(kBfMaxWarps * 32)
    bf16_gemv16_kernel(const uint16_t *__restrict__ w_a, const uint16_t *__restrict__ w_b,
                       const uint16_t *__restrict__ x, uint16_t *__restrict__ y_bf16, float *__restrict__ y_f32,
                       int rows, int cols, int T) {
  extern __shared__ __align__(16) unsigned char smem[];
  __shared__ float partial[kBfMaxWarps][16][8];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarps = blockDim.x >> 5;
  const int g = lane >> 2, t = lane & 3;
  stage_x_bf16(x, smem, cols, T, tid, blockDim.x);
  __syncthreads();
  const size_t wrow = cols / 8;  // uint4 per row
  const uint4 *w_lo, *w_hi;
  if (MODE == 0) {
    const int row0 = blockIdx.x * 16;
    w_lo = reinterpret_cast<const uint4 *>(w_a) + (size_t)(row0 + g) * wrow;
    w_hi = w_lo + 8 * wrow;
  } else {
    const int row0 = blockIdx.x * 8;
    w_lo = reinterpret_cast<const uint4 *>(w_a) + (size_t)(row0 + g) * wrow;
    w_hi = reinterpret_cast<const uint4 *>(w_b) + (size_t)(row0 + g) * wrow;
  }
  const int tok = g < T ? g : T - 1;
  const uint4 *xrow = reinterpret_cast<const uint4 *>(smem + tok * bf16_x_row_bytes(cols)) + t;
  // k-steps split as evenly as possible over the warps
  const int ksteps = cols / 32;
  const int base = ksteps / nwarps, rem = ksteps % nwarps;
  const int ks0 = warp * base + (warp < rem ? warp : rem);
  const int nsteps = base + (warp < rem ? 1 : 0);
  float d[4] = {0.f, 0.f, 0.f, 0.f};
  bf16_rows16_accumulate(w_lo, w_hi, xrow, ks0, nsteps, t, d);
  partial[warp][g][2 * t] = d[0];
  partial[warp][g][2 * t + 1] = d[1];
  partial[warp][g + 8][2 * t] = d[2];
  partial[warp][g + 8][2 * t + 1] = d[3];
  __syncthreads();
  if (MODE == 0) {
    if (tid < 16 * 8) {
      int r = tid >> 3, tk = tid & 7;
      if (tk < T) {
        float v = 0.f;
        for (int wi = 0; wi < nwarps; ++wi) v += partial[wi][r][tk];
        size_t o = (size_t)tk * rows + blockIdx.x * 16 + r;
        if (y_f32) y_f32[o] = v;
        else y_bf16[o] = f32_to_bf16_bits(v);
      }
    }
  } else {
    if (tid < 8 * 8) {
      int r = tid >> 3, tk = tid & 7;
      if (tk < T) {
        float gv = 0.f, uv = 0.f;
        for (int wi = 0; wi < nwarps; ++wi) {
          gv += partial[wi][r][tk];
          uv += partial[wi][r + 8][tk];
        }
        gv = round_bf16(gv);
        uv = round_bf16(uv);
        float m = round_bf16(round_bf16(gv / (1.0f + expf(-gv))) * uv);
        y_bf16[(size_t)tk * rows + blockIdx.x * 8 + r] = f32_to_bf16_bits(m);
      }
    }
  }
}

// Scalar fallback: one warp per (row, token); cols % 8 == 0, any rows.
__global__ void bf16_gemv_scalar_kernel(const uint16_t *__restrict__ w, const uint16_t *__restrict__ x,
                                        uint16_t *__restrict__ y_bf16, float *__restrict__ y_f32, int rows, int cols,
                                        int T) {
  int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (warp >= rows) return;
  const uint4 *wr = reinterpret_cast<const uint4 *>(w + (size_t)warp * cols);
  for (int tk = 0; tk < T; ++tk) {
    const uint4 *xr = reinterpret_cast<const uint4 *>(x + (size_t)tk * cols);
    float acc = 0.f;
    for (int c = lane; c < cols / 8; c += 32) {
      uint4 a = ldg_stream(wr + c), b = xr[c];
      acc = fmaf(bf16lo(a.x), bf16lo(b.x), acc);
      acc = fmaf(bf16hi(a.x), bf16hi(b.x), acc);
      acc = fmaf(bf16lo(a.y), bf16lo(b.y), acc);
      acc = fmaf(bf16hi(a.y), bf16hi(b.y), acc);
      acc = fmaf(bf16lo(a.z), bf16lo(b.z), acc);
      acc = fmaf(bf16hi(a.z), bf16hi(b.z), acc);
      acc = fmaf(bf16lo(a.w), bf16lo(b.w), acc);
      acc = fmaf(bf16hi(a.w), bf16hi(b.w), acc);
    }
    acc = warp_sum(acc);
    if (lane == 0) {
      if (y_f32) y_f32[(size_t)tk * rows + warp] = acc;
      else y_bf16[(size_t)tk * rows + warp] = f32_to_bf16_bits(acc);
    }
  }
}

// Split-K form of the plain mat-vec for matrices with few rows (q_a 1536, kv_a 576 rows): grid = (rows / 16, ksplit),
// so that every SM streams weights whatever the row count, and a CTA stages only its own K-range of the
// activations.  Partial sums go to `part` ([ksplit][rows / 16][16][8] fp32); the CTA that draws the last ticket of a
// row block adds them in split order (deterministic) and writes the rounded result, then re-arms the ticket.
// STAGE false: the activations are not copied to shared memory at all; every lane reads its token's 16 bytes of a k-step
// straight from global memory, which the L1 keeps (the weights bypass it).  With more than two tokens a CTA's staged
// slice is no longer small against its 16 weight rows, and without shared memory more CTAs fit on an SM.
template <bool STAGE>
__global__ void __launch_bounds__(128) bf16_gemv16_splitk_kernel(const uint16_t *__restrict__ w, const uint16_t *__restrict__ x,
                                                                 uint16_t *__restrict__ y_bf16, float *__restrict__ y_f32,
                                                                 int rows, int cols, int T, int ksteps_per_split,
                                                                 float *__restrict__ part, unsigned *__restrict__ tickets,
                                                                 const uint16_t *__restrict__ w2, uint16_t *__restrict__ y2_bf16,
                                                                 int rows2) {
  extern __shared__ __align__(16) unsigned char smem[];
  __shared__ float partial[4][16][8];
  __shared__ unsigned s_ticket;
  // w2 != NULL: a second matrix over the same activations in the same launch (q_a and kv_a of the attention block);
  // its row blocks follow the first matrix's in blockIdx.x
  int rbx = blockIdx.x;
  if (w2 && rbx >= rows / 16) {
    rbx -= rows / 16;
    w = w2;
    y_bf16 = y2_bf16;
    y_f32 = nullptr;
    rows = rows2;
  }
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int ksteps = cols / 32;
  const int kbeg = blockIdx.y * ksteps_per_split;
  const int kn = min(ksteps_per_split, ksteps - kbeg);  // k-steps of this CTA
  // stage x[:, 32 kbeg .. 32 (kbeg + kn)) with the row skew of stage_x_bf16
  const int per_row = kn * 4;  // uint4 per token row
  const size_t row_bytes = bf16_x_row_bytes(kn * 32);
  if (STAGE) {
    for (int u = tid; u < per_row * T; u += blockDim.x) {
      const int tok = u / per_row, c = u - tok * per_row;
      reinterpret_cast<uint4 *>(smem + tok * row_bytes)[c] = reinterpret_cast<const uint4 *>(x + (size_t)tok * cols)[kbeg * 4 + c];
    }
    __syncthreads();
  }
  const size_t wrow = cols / 8;
  const uint4 *w_lo = reinterpret_cast<const uint4 *>(w) + (size_t)(rbx * 16 + g) * wrow + (size_t)kbeg * 4;
  const uint4 *w_hi = w_lo + 8 * wrow;
  const int tok = g < T ? g : T - 1;
  const uint4 *xrow = STAGE ? reinterpret_cast<const uint4 *>(smem + tok * row_bytes) + t
                            : reinterpret_cast<const uint4 *>(x + (size_t)tok * cols) + (size_t)kbeg * 4 + t;
  const int base = kn / 4, rem = kn % 4;
  const int ks0 = warp * base + (warp < rem ? warp : rem);
  const int nsteps = base + (warp < rem ? 1 : 0);
  float d[4] = {0.f, 0.f, 0.f, 0.f};
  bf16_rows16_accumulate(w_lo, w_hi, xrow, ks0, nsteps, t, d);
  partial[warp][g][2 * t] = d[0];
  partial[warp][g][2 * t + 1] = d[1];
  partial[warp][g + 8][2 * t] = d[2];
  partial[warp][g + 8][2 * t + 1] = d[3];
  __syncthreads();
  const int r = tid >> 3, tk = tid & 7;  // 128 threads = 16 rows x 8 tokens
  float v = (partial[0][r][tk] + partial[1][r][tk]) + (partial[2][r][tk] + partial[3][r][tk]);
  const int nsplit = gridDim.y;
  if (nsplit > 1) {
    part[((size_t)blockIdx.y * gridDim.x + blockIdx.x) * 128 + tid] = v;
    __threadfence();
    __syncthreads();
    if (tid == 0) s_ticket = atomicAdd(tickets + blockIdx.x, 1u);
    __syncthreads();
    if (s_ticket != (unsigned)nsplit - 1) return;
    __threadfence();
    v = 0.f;
    for (int sidx = 0; sidx < nsplit; ++sidx) v += __ldcg(part + ((size_t)sidx * gridDim.x + blockIdx.x) * 128 + tid);
    if (tid == 0) tickets[blockIdx.x] = 0;
  }
  if (tk < T) {
    const size_t o = (size_t)tk * rows + rbx * 16 + r;
    if (y_f32) y_f32[o] = v;
    else y_bf16[o] = f32_to_bf16_bits(v);
  }
}

// One CTA per token.  The row is read once with 16-byte loads, all of them in flight before the first use (a row of
// up to 256 x 4 x 8 = 8192 values stays in registers between the sum and the scaling); longer or unaligned rows take
// the element loop.
// ADD: first x <- bf16(x + t) (the rounded residual add, src/kimi_exec.cu:248-251), written back, then the norm of it.
template <bool ADD>
__global__ void __launch_bounds__(256) rmsnorm_kernel(uint16_t *__restrict__ x, const uint16_t *__restrict__ tadd,
                                                      const uint16_t *__restrict__ w, uint16_t *__restrict__ y, int n, float eps) {
  __shared__ float red[32];
  uint16_t *xr = x + (size_t)blockIdx.x * n;
  const uint16_t *tr = ADD ? tadd + (size_t)blockIdx.x * n : nullptr;
  uint16_t *yr = y + (size_t)blockIdx.x * n;
  const bool vec = (n % 8 == 0) && n <= 8192 && ((reinterpret_cast<uintptr_t>(xr) | reinterpret_cast<uintptr_t>(yr) |
                                                  reinterpret_cast<uintptr_t>(w) | reinterpret_cast<uintptr_t>(tr)) & 15) == 0;
  float v = 0.f;
  uint4 xv[4];
  const int nu = n / 8;
  if (vec) {
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const int u = threadIdx.x + k * 256;
      xv[k] = u < nu ? reinterpret_cast<const uint4 *>(xr)[u] : make_uint4(0, 0, 0, 0);
      if (ADD && u < nu) {
        const uint4 tv = reinterpret_cast<const uint4 *>(tr)[u];
        const uint32_t a[4] = {xv[k].x, xv[k].y, xv[k].z, xv[k].w}, c[4] = {tv.x, tv.y, tv.z, tv.w};
        uint32_t o[4];
#pragma unroll
        for (int j = 0; j < 4; ++j)
          o[j] = f32_to_bf16_bits(bf16lo(a[j]) + bf16lo(c[j])) | ((uint32_t)f32_to_bf16_bits(bf16hi(a[j]) + bf16hi(c[j])) << 16);
        xv[k] = make_uint4(o[0], o[1], o[2], o[3]);
        reinterpret_cast<uint4 *>(xr)[u] = xv[k];
      }
    }
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const uint32_t q[4] = {xv[k].x, xv[k].y, xv[k].z, xv[k].w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float lo = bf16lo(q[j]), hi = bf16hi(q[j]);
        v = fmaf(lo, lo, v);
        v = fmaf(hi, hi, v);
      }
    }
  } else {
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
      if (ADD) xr[i] = f32_to_bf16_bits(bf16_bits_to_f32(xr[i]) + bf16_bits_to_f32(tr[i]));
      float a = bf16_bits_to_f32(xr[i]);
      v = fmaf(a, a, v);
    }
  }
  v = warp_sum(v);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  if (threadIdx.x < 32) {
    float s = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : 0.f;
    s = warp_sum(s);
    if (threadIdx.x == 0) red[0] = s;
  }
  __syncthreads();
  const float scale = rsqrtf(red[0] / n + eps);
  if (vec) {
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const int u = threadIdx.x + k * 256;
      if (u < nu) {
        const uint4 wv = reinterpret_cast<const uint4 *>(w)[u];
        const uint32_t q[4] = {xv[k].x, xv[k].y, xv[k].z, xv[k].w}, ww[4] = {wv.x, wv.y, wv.z, wv.w};
        uint32_t o[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const uint32_t lo = f32_to_bf16_bits(round_bf16(bf16lo(q[j]) * scale) * bf16lo(ww[j]));
          const uint32_t hi = f32_to_bf16_bits(round_bf16(bf16hi(q[j]) * scale) * bf16hi(ww[j]));
          o[j] = lo | (hi << 16);
        }
        reinterpret_cast<uint4 *>(yr)[u] = make_uint4(o[0], o[1], o[2], o[3]);
      }
    }
  } else {
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
      float a = bf16_bits_to_f32(xr[i]);
      yr[i] = f32_to_bf16_bits(round_bf16(a * scale) * bf16_bits_to_f32(w[i]));
    }
  }
}
__global__ void add_bf16_kernel(uint16_t *__restrict__ a, const uint16_t *__restrict__ b, long n) {
  long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) a[i] = f32_to_bf16_bits(bf16_bits_to_f32(a[i]) + bf16_bits_to_f32(b[i]));
}

static bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

int launch_bf16_gemv(const uint16_t *w, const uint16_t *x, uint16_t *y_bf16, float *y_f32, int rows, int cols, int T,
                     cudaStream_t stream) {
  size_t smem = bf16_x_row_bytes(cols) * T;
  bool tc = rows % 16 == 0 && cols % 32 == 0 && aligned16(w) && aligned16(x) && smem <= 200 * 1024;
  if (tc) {
    if (smem > 48 * 1024)
      BLOK_CUDA(cudaFuncSetAttribute(bf16_gemv16_kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    int nwarps = cols >= 4096 ? 16 : (cols >= 1024 ? 8 : 4);
    bf16_gemv16_kernel<0><<<rows / 16, nwarps * 32, smem, stream>>>(w, nullptr, x, y_bf16, y_f32, rows, cols, T);
    return launch_status("bf16_gemv16_kernel");
  }
  bf16_gemv_scalar_kernel<<<(rows + 7) / 8, 256, 0, stream>>>(w, x, y_bf16, y_f32, rows, cols, T);
  return launch_status("bf16_gemv_scalar_kernel");
}

// Bytes of workspace launch_bf16_gemv_splitk may need for a matrix of `rows` rows: one ticket per row block at the
// start (the same words serve every matrix that uses the workspace; they re-arm themselves), then 512 bytes of
// partial sums per CTA (splits x row blocks < 4 SMs' worth + row blocks).
static size_t splitk_ticket_bytes(int rows) { return ((size_t)(rows / 16) * 4 + 255) / 256 * 256; }
size_t bf16_gemv_splitk_workspace_bytes(int rows) {
  return splitk_ticket_bytes(rows) + ((size_t)4 * sm_count() + rows / 16) * 128 * 4;
}

// The mat-vec with as many K-splits as it takes to put about four CTAs on every SM; falls back to the one-CTA-per-
// row-block kernel when the matrix has enough rows or the shape does not fit.  `ws` must be zero before the first call
// (the tickets re-arm themselves) and is used by one launch at a time.
int launch_bf16_gemv_splitk(const uint16_t *w, const uint16_t *x, uint16_t *y_bf16, float *y_f32, int rows, int cols, int T,
                            void *ws, size_t ws_bytes, cudaStream_t stream) {
  const int rb = rows / 16, ksteps = cols / 32;
  int ksplit = rb > 0 ? (4 * sm_count() + rb - 1) / rb : 1;
  ksplit = std::min(ksplit, std::min(32, ksteps / 8));
  const bool ok = rows % 16 == 0 && cols % 32 == 0 && (reinterpret_cast<uintptr_t>(w) & 15) == 0 &&
                  (reinterpret_cast<uintptr_t>(x) & 15) == 0 && T >= 1 && T <= 8 && ws &&
                  ws_bytes >= bf16_gemv_splitk_workspace_bytes(rows);
  if (!ok || (ksplit < 2 && T <= 2)) return launch_bf16_gemv(w, x, y_bf16, y_f32, rows, cols, T, stream);
  ksplit = std::max(ksplit, 1);
  const int per = (ksteps + ksplit - 1) / ksplit;
  ksplit = (ksteps + per - 1) / per;
  // the ticket block is sized for the largest matrix the workspace was made for; this matrix uses its first rb words
  unsigned *tickets = static_cast<unsigned *>(ws);
  float *part = reinterpret_cast<float *>(static_cast<unsigned char *>(ws) + (ws_bytes - ((size_t)4 * sm_count() + rb) * 128 * 4) / 256 * 256);
  if (T > 2) {  // activations through the L1, no shared memory
    bf16_gemv16_splitk_kernel<false><<<dim3(rb, ksplit), 128, 0, stream>>>(w, x, y_bf16, y_f32, rows, cols, T, per, part, tickets, nullptr,
                                                                           nullptr, 0);
    return launch_status("bf16_gemv16_splitk_kernel<l1>");
  }
  const size_t smem = bf16_x_row_bytes(per * 32) * T;
  if (smem > 48 * 1024)
    BLOK_CUDA(cudaFuncSetAttribute(bf16_gemv16_splitk_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  bf16_gemv16_splitk_kernel<true><<<dim3(rb, ksplit), 128, smem, stream>>>(w, x, y_bf16, y_f32, rows, cols, T, per, part, tickets, nullptr,
                                                                           nullptr, 0);
  return launch_status("bf16_gemv16_splitk_kernel");
}

// Two matrices over the same activations in ONE launch (y1 = W1 x, y2 = W2 x, both bf16): the row blocks of the second
// follow those of the first in the grid.  `ws` as for launch_bf16_gemv_splitk with rows = rows1 + rows2.  Falls back to
// two launches where the single one does not apply.
int launch_bf16_gemv_splitk_pair(const uint16_t *w1, int rows1, uint16_t *y1, const uint16_t *w2, int rows2, uint16_t *y2,
                                 const uint16_t *x, int cols, int T, void *ws, size_t ws_bytes, cudaStream_t stream) {
  const int rb = (rows1 + rows2) / 16, ksteps = cols / 32;
  int ksplit = rb > 0 ? (4 * sm_count() + rb - 1) / rb : 1;
  ksplit = std::max(1, std::min(ksplit, std::min(32, ksteps / 8)));
  const bool ok = rows1 % 16 == 0 && rows2 % 16 == 0 && cols % 32 == 0 && (reinterpret_cast<uintptr_t>(w1) & 15) == 0 &&
                  (reinterpret_cast<uintptr_t>(w2) & 15) == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0 && T >= 1 && T <= 8 && ws &&
                  ws_bytes >= bf16_gemv_splitk_workspace_bytes(rows1 + rows2);
  if (!ok) {
    if (int rc = launch_bf16_gemv_splitk(w1, x, y1, nullptr, rows1, cols, T, ws, ws_bytes, stream)) return rc;
    return launch_bf16_gemv_splitk(w2, x, y2, nullptr, rows2, cols, T, ws, ws_bytes, stream);
  }
  const int per = (ksteps + ksplit - 1) / ksplit;
  ksplit = (ksteps + per - 1) / per;
  unsigned *tickets = static_cast<unsigned *>(ws);
  float *part = reinterpret_cast<float *>(static_cast<unsigned char *>(ws) + (ws_bytes - ((size_t)4 * sm_count() + rb) * 128 * 4) / 256 * 256);
  if (T > 2) {
    bf16_gemv16_splitk_kernel<false><<<dim3(rb, ksplit), 128, 0, stream>>>(w1, x, y1, nullptr, rows1, cols, T, per, part, tickets, w2, y2, rows2);
    return launch_status("bf16_gemv16_splitk_kernel<l1, pair>");
  }
  const size_t smem = bf16_x_row_bytes(per * 32) * T;
  if (smem > 48 * 1024)
    BLOK_CUDA(cudaFuncSetAttribute(bf16_gemv16_splitk_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  bf16_gemv16_splitk_kernel<true><<<dim3(rb, ksplit), 128, smem, stream>>>(w1, x, y1, nullptr, rows1, cols, T, per, part, tickets, w2, y2, rows2);
  return launch_status("bf16_gemv16_splitk_kernel<pair>");
}


// mid[T, ffn] = SwiGLU front half.
int launch_bf16_gateup(const uint16_t *gate, const uint16_t *up, const uint16_t *x, uint16_t *mid, int ffn, int cols,
                       int T, cudaStream_t stream) {
  size_t smem = bf16_x_row_bytes(cols) * T;
  if (smem > 48 * 1024)
    BLOK_CUDA(cudaFuncSetAttribute(bf16_gemv16_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  int nwarps = cols >= 4096 ? 16 : (cols >= 1024 ? 8 : 4);
  bf16_gemv16_kernel<1><<<ffn / 8, nwarps * 32, smem, stream>>>(gate, up, x, mid, nullptr, ffn, cols, T);
  return launch_status("bf16_gemv16_kernel<swiglu>");
}

}  // namespace blok

using namespace blok;

extern "C" int blok_bf16_gemv(const blok_bf16_t *w, const blok_bf16_t *x, blok_bf16_t *y_bf16, float *y_f32, int rows,
                              int cols, int T, blok_stream_t stream) {
  BLOK_REQUIRE(w && x && ((y_bf16 != nullptr) != (y_f32 != nullptr)), BLOK_ERR_ARG,
               "blok_bf16_gemv: need w, x and exactly one of y_bf16 / y_f32");
  BLOK_REQUIRE(rows >= 0 && cols > 0 && cols % 8 == 0 && T >= 1 && T <= 8, BLOK_ERR_SHAPE,
               "blok_bf16_gemv: cols %d must be a positive multiple of 8 and 1 <= T=%d <= 8", cols, T);
  BLOK_REQUIRE(aligned16(w) && aligned16(x), BLOK_ERR_ARG, "blok_bf16_gemv: w and x must be 16-byte aligned");
  if (rows == 0) return BLOK_OK;
  return launch_bf16_gemv(w, x, y_bf16, y_f32, rows, cols, T, (cudaStream_t)stream);
}

// mid [T, ffn] bf16, then (more than 8 rows) the K-split partial sums of the down projection
static size_t mlp_mid_bytes(int ffn, int T) { return ((size_t)ffn * T * sizeof(uint16_t) + 255) / 256 * 256; }
extern "C" size_t blok_bf16_mlp_workspace_bytes(int hidden, int ffn, int T) {
  if (ffn <= 0 || T <= 0) return 0;
  if (T <= 8) return (size_t)ffn * T * sizeof(uint16_t);
  return mlp_mid_bytes(ffn, T) + std::max(wgemm_splitk_bytes(WG_BF16_SWIGLU, hidden, ffn, T), wgemm_splitk_bytes(WG_BF16_PLAIN, ffn, hidden, T));
}

extern "C" int blok_bf16_mlp(const blok_bf16_t *gate, const blok_bf16_t *up, const blok_bf16_t *down,
                             const blok_bf16_t *x, blok_bf16_t *y, int hidden, int ffn, int T, void *workspace,
                             size_t workspace_bytes, blok_stream_t stream) {
  BLOK_REQUIRE(gate && up && down && x && y && workspace, BLOK_ERR_ARG, "blok_bf16_mlp: null pointer");
  BLOK_REQUIRE(hidden > 0 && ffn > 0 && hidden % 32 == 0 && ffn % 32 == 0 && hidden % 16 == 0 && T >= 1 && T <= kWgStreamTokens,
               BLOK_ERR_SHAPE, "blok_bf16_mlp: hidden %d, ffn %d must be multiples of 32 and 1 <= T=%d <= %d", hidden, ffn, T,
               kWgStreamTokens);
  BLOK_REQUIRE(T <= 8 || (hidden % 256 == 0 && ffn % 256 == 0), BLOK_ERR_SHAPE,
               "blok_bf16_mlp: more than 8 rows need hidden %d and ffn %d to be multiples of 256", hidden, ffn);
  BLOK_REQUIRE(T > 8 || bf16_x_row_bytes(hidden > ffn ? hidden : ffn) * T <= 200 * 1024, BLOK_ERR_SHAPE,
               "blok_bf16_mlp: T * max(hidden, ffn) does not fit in shared memory");
  BLOK_REQUIRE(workspace_bytes >= blok_bf16_mlp_workspace_bytes(hidden, ffn, T), BLOK_ERR_WORKSPACE,
               "blok_bf16_mlp: workspace too small");
  BLOK_REQUIRE(aligned16(gate) && aligned16(up) && aligned16(down) && aligned16(x) && aligned16(workspace), BLOK_ERR_ARG,
               "blok_bf16_mlp: pointers must be 16-byte aligned");
  uint16_t *mid = static_cast<uint16_t *>(workspace);
  if (T > 8) {  // 9..64 rows: each matrix streamed once for all rows (wgemm_stream.cu)
    float *sk = reinterpret_cast<float *>(static_cast<unsigned char *>(workspace) + mlp_mid_bytes(ffn, T));
    const size_t sk_bytes = workspace_bytes - mlp_mid_bytes(ffn, T);
    if (int rc = launch_wgemm_rows(WG_BF16_SWIGLU, gate, up, x, mid, nullptr, ffn, hidden, T, sk, sk_bytes, (cudaStream_t)stream)) return rc;
    return launch_wgemm_rows(WG_BF16_PLAIN, down, nullptr, mid, y, nullptr, hidden, ffn, T, sk, sk_bytes, (cudaStream_t)stream);
  }
  int rc = launch_bf16_gateup(gate, up, x, mid, ffn, hidden, T, (cudaStream_t)stream);
  if (rc) return rc;
  return launch_bf16_gemv(down, mid, y, nullptr, hidden, ffn, T, (cudaStream_t)stream);
}

extern "C" int blok_rmsnorm(const blok_bf16_t *x, const blok_bf16_t *w, blok_bf16_t *y, int T, int n, float eps,
                            blok_stream_t stream) {
  BLOK_REQUIRE(x && w && y, BLOK_ERR_ARG, "blok_rmsnorm: null pointer");
  BLOK_REQUIRE(T >= 0 && n > 0, BLOK_ERR_SHAPE, "blok_rmsnorm: bad shape T=%d n=%d", T, n);
  if (T == 0) return BLOK_OK;
  rmsnorm_kernel<false><<<T, 256, 0, (cudaStream_t)stream>>>(const_cast<uint16_t *>(x), nullptr, w, y, n, eps);
  return launch_status("rmsnorm_kernel");
}

extern "C" int blok_add_rmsnorm(blok_bf16_t *x, const blok_bf16_t *t, const blok_bf16_t *w, blok_bf16_t *y, int T, int n,
                                float eps, blok_stream_t stream) {
  BLOK_REQUIRE(x && t && w && y, BLOK_ERR_ARG, "blok_add_rmsnorm: null pointer");
  BLOK_REQUIRE(T >= 0 && n > 0, BLOK_ERR_SHAPE, "blok_add_rmsnorm: bad shape T=%d n=%d", T, n);
  if (T == 0) return BLOK_OK;
  rmsnorm_kernel<true><<<T, 256, 0, (cudaStream_t)stream>>>(x, t, w, y, n, eps);
  return launch_status("rmsnorm_kernel<add>");
}

extern "C" int blok_add_bf16(blok_bf16_t *a, const blok_bf16_t *b, long n, blok_stream_t stream) {
  BLOK_REQUIRE(a && b, BLOK_ERR_ARG, "blok_add_bf16: null pointer");
  BLOK_REQUIRE(n >= 0, BLOK_ERR_SHAPE, "blok_add_bf16: negative n");
  if (n == 0) return BLOK_OK;
  add_bf16_kernel<<<(unsigned)((n + 255) / 256), 256, 0, (cudaStream_t)stream>>>(a, b, n);
  return launch_status("add_bf16_kernel");
}
