// Warp-level top-k selection of the router (one warp per token).
#pragma once
#include <cmath>

#include "common.cuh"

namespace blok {

// score/sel: shared-memory arrays of `experts` floats owned by this warp, already
// filled with s = sigmoid(logit) and sel = s + bias (and __syncwarp()ed).  Runs
// `topk` rounds of argmax over sel with the reference's rule (strict '>' scanning
// ascending indices: the lowest index wins a tie; src/kimi_exec.cu:390-395).
// Lane k < topk returns the k-th selected expert in my_id and its normalised,
// scaled weight in my_w.
__device__ __forceinline__ void warp_topk(const float *score, float *sel, int experts, int topk, float routed_scale,
                                          int lane, int &my_id, float &my_w) {
  float sum = 0.f;
  my_w = 0.f;
  my_id = 0;
  for (int k = 0; k < topk; ++k) {
    float best = -INFINITY;
    int id = 0x7fffffff;
    for (int i = lane; i < experts; i += 32) {
      float v = sel[i];
      if (v > best) best = v, id = i;
    }
#pragma unroll
    for (int o = 16; o; o >>= 1) {
      float ob = __shfl_xor_sync(0xffffffffu, best, o);
      int oi = __shfl_xor_sync(0xffffffffu, id, o);
      if (ob > best || (ob == best && oi < id)) best = ob, id = oi;
    }
    if (id == 0x7fffffff) id = 0;  // every candidate was -inf or NaN: the reference keeps id 0
    float s = score[id];
    sum += s;
    if (lane == k) my_w = s, my_id = id;
    __syncwarp();
    if (lane == 0) sel[id] = -INFINITY;
    __syncwarp();
  }
  my_w = my_w / (sum + 1.0e-20f) * routed_scale;
}

}  // namespace blok
