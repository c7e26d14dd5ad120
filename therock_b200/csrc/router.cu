// Router: logits [T, E] -> top-K expert ids and renormalised weights, one warp per token.
// Scores are softmax(logits) or sigmoid(logits) in f32; the K largest are taken with ties
// going to the lower expert index; the K weights are divided by their sum.  The outputs are
// exactly what moe_sorting / fused_moe consume, so a layer can go logits -> fused_moe with
// no host step in between.
#include <cuda_runtime.h>

#include "../../include/fused_moe_c.h"
#include "plan.hpp"

namespace fmoe {
namespace {

constexpr int kRouteWarps = 8;
constexpr int kMaxPerLane = 32;   // experts per lane: E <= 1024

__global__ void __launch_bounds__(kRouteWarps * 32)
route_kernel(const float* __restrict__ logits, int T, int E, int K, int mode,
             int32_t* __restrict__ ids, float* __restrict__ weights) {
  const int lane = threadIdx.x & 31;
  const int t = blockIdx.x * kRouteWarps + (threadIdx.x >> 5);
  if (t >= T) return;
  const float* l = logits + static_cast<size_t>(t) * E;
  float s[kMaxPerLane];
  const int per_lane = (E + 31) >> 5;
  // lane owns experts lane, lane+32, ... (coalesced loads)
  float mx = -INFINITY;
#pragma unroll
  for (int j = 0; j < kMaxPerLane; ++j) {
    const int e = lane + 32 * j;
    s[j] = (j < per_lane && e < E) ? l[e] : -INFINITY;
    mx = fmaxf(mx, s[j]);
  }
  if (mode == 0) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
    float sum = 0.0f;
#pragma unroll
    for (int j = 0; j < kMaxPerLane; ++j) {
      const int e = lane + 32 * j;
      if (j < per_lane && e < E) { s[j] = expf(s[j] - mx); sum += s[j]; }
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
#pragma unroll
    for (int j = 0; j < kMaxPerLane; ++j) {
      const int e = lane + 32 * j;
      if (j < per_lane && e < E) s[j] = s[j] / sum;
    }
  } else {
#pragma unroll
    for (int j = 0; j < kMaxPerLane; ++j) {
      const int e = lane + 32 * j;
      if (j < per_lane && e < E) s[j] = 1.0f / (1.0f + expf(-s[j]));
    }
  }
  float total = 0.0f;
  float my_w = 0.0f;      // lane k keeps the k-th selected weight
  int my_id = 0;
  for (int k = 0; k < K; ++k) {
    // local best among this lane's unselected experts (selected ones are set to -inf)
    float bv = -INFINITY;
    int be = 0x7fffffff;
#pragma unroll
    for (int j = 0; j < kMaxPerLane; ++j) {
      const int e = lane + 32 * j;
      if (j < per_lane && e < E && (s[j] > bv)) { bv = s[j]; be = e; }   // ascending e: first max wins
    }
    // warp arg-max, ties to the lower index
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, off);
      const int oe = __shfl_xor_sync(0xffffffffu, be, off);
      if (ov > bv || (ov == bv && oe < be)) { bv = ov; be = oe; }
    }
    if ((be & 31) == lane) {
#pragma unroll
      for (int j = 0; j < kMaxPerLane; ++j)
        if (lane + 32 * j == be) s[j] = -INFINITY;
    }
    if (lane == (k & 31)) { my_w = bv; my_id = be; }
    total += bv;
  }
  // K <= 32: lane k holds selection k; renormalise and store
  if (lane < K) {
    ids[static_cast<size_t>(t) * K + lane] = my_id;
    weights[static_cast<size_t>(t) * K + lane] = my_w / total;
  }
}

}  // namespace
}  // namespace fmoe

extern "C" int fmoe_route(const float* logits, int32_t T, int32_t E, int32_t K, int32_t mode,
                          int32_t* topk_ids, float* topk_weight, void* stream) {
  if (!logits || !topk_ids || !topk_weight)
    return fmoe::fail(FMOE_ERR_INVALID_ARG, "fmoe_route: logits, topk_ids and topk_weight are required");
  if (T < 0 || E <= 0 || K <= 0 || K > E || (mode != 0 && mode != 1))
    return fmoe::fail(FMOE_ERR_INVALID_ARG, "fmoe_route: bad arguments (T=%d E=%d K=%d mode=%d)", T, E, K, mode);
  if (E > 32 * fmoe::kMaxPerLane || K > 32)
    return fmoe::fail(FMOE_ERR_UNSUPPORTED, "fmoe_route: at most %d experts and 32 experts per token", 32 * fmoe::kMaxPerLane);
  if (T == 0) return FMOE_OK;
  const int grid = (T + fmoe::kRouteWarps - 1) / fmoe::kRouteWarps;
  fmoe::route_kernel<<<grid, fmoe::kRouteWarps * 32, 0, static_cast<cudaStream_t>(stream)>>>(
      logits, T, E, K, mode, topk_ids, topk_weight);
  const cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? FMOE_OK : fmoe::fail(FMOE_ERR_CUDA, "fmoe_route launch failed: %s", cudaGetErrorString(e));
}
