// moe_sorting for sm_100a: stable bucketing of the T*K routed (token, k) pairs by expert,
// every bucket padded to a multiple of block_m.
//
// One CTA of 32 warps.  The flat pair range is cut into 32 contiguous chunks, one per
// warp, so the stable order inside an expert is (chunk, position in chunk).  Pass 1 counts
// per (warp, expert) with __match_any_sync groups; a warp-shuffle prefix sum over the
// experts turns the counts into padded bucket offsets; pass 2 re-walks the chunks and
// places every pair at  offset[e] + (pairs of e in earlier chunks) + (rank inside the
// 32-wide group, from the match mask).  All arithmetic is integer: the result is
// bit-exact by construction.
#include "internal.h"
#include "ptx.cuh"

namespace fmoe {
namespace {

constexpr int kSortThreads = 1024;
constexpr int kSortWarps = kSortThreads / 32;
constexpr int kSortMaxCtas = 64;                 // CTAs of the multi-CTA path
constexpr int kSortMultiCtaMinPairs = 8192;      // below this one CTA is faster (one launch)

__global__ void __launch_bounds__(kSortThreads, 1)
moe_sorting_kernel(const int32_t* __restrict__ topk_ids, const float* __restrict__ topk_weight,
                   int T_max, const int32_t* __restrict__ num_tokens_dev, int K, int E, int id_div,
                   int block_m, int cap,
                   int32_t* __restrict__ sorted_token_ids, float* __restrict__ sorted_weights,
                   int32_t* __restrict__ sorted_rows, int32_t* __restrict__ sorted_expert_ids,
                   int32_t* __restrict__ num_post_pad, int32_t* __restrict__ mblk_cum,
                   int32_t* __restrict__ status_to_clear, int32_t* __restrict__ inv_out) {
  ptx::pdl_wait();      // inputs may come from the kernel just before this one
  ptx::pdl_release();
  extern __shared__ int32_t sm[];
  int32_t* cnt = sm;                      // [kSortWarps][E] counts, later running offsets
  int32_t* blk_cum = sm + kSortWarps * E; // [E + 1] cumulative padded blocks
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  // the token count may live on the device (expert-parallel receive side); T_max bounds it
  const int T = num_tokens_dev ? min(T_max, max(0, *num_tokens_dev)) : T_max;
  const int R = T * K;
  const int id_limit = E * id_div;       // bucket = id / id_div (id_div > 1: bucket by owner rank)
  // chunk length: multiple of 32 so every warp iterates over whole 32-wide groups
  const int chunk = ((R + kSortWarps - 1) / kSortWarps + 31) & ~31;
  const int r_begin = warp * chunk;
  const int r_end = min(R, r_begin + chunk);

  for (int i = tid; i < kSortWarps * E; i += kSortThreads) cnt[i] = 0;
  for (int i = tid; i < cap; i += kSortThreads) {
    sorted_token_ids[i] = T_max;
    if (sorted_weights) sorted_weights[i] = 0.0f;
    if (sorted_rows) sorted_rows[i] = -1;
  }
  if (sorted_expert_ids)
    for (int i = tid; i < cap / block_m; i += kSortThreads) sorted_expert_ids[i] = -1;
  __syncthreads();

  // pass 1: per-(warp, expert) histogram.  Four 32-wide groups are loaded before any is
  // processed so the global-load latency is paid once per 128 pairs, not once per 32.
  constexpr int kUnroll = 4;
  int32_t* my_cnt = cnt + warp * E;
  for (int r0 = r_begin; r0 < r_end; r0 += 32 * kUnroll) {
    int ev[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const int r = r0 + u * 32 + lane;
      ev[u] = (r < r_end) ? topk_ids[r] : -1;
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      if (r0 + u * 32 >= r_end) break;               // warp-uniform
      int e = ev[u];
      e = (e < 0 || e >= id_limit) ? -1 : e / id_div;
      const unsigned mask = __match_any_sync(0xffffffffu, e);
      if (e >= 0 && lane == (__ffs(mask) - 1)) my_cnt[e] += __popc(mask);
      __syncwarp();
    }
  }
  __syncthreads();

  // per expert: total, and counts -> exclusive prefix over warps
  for (int e = tid; e < E; e += kSortThreads) {
    int run = 0;
    for (int w = 0; w < kSortWarps; ++w) {
      const int c = cnt[w * E + e];
      cnt[w * E + e] = run;
      run += c;
    }
    blk_cum[e + 1] = (run + block_m - 1) / block_m;   // padded blocks of expert e
  }
  if (tid == 0) blk_cum[0] = 0;
  __syncthreads();

  // inclusive prefix sum of the block counts over experts: warp 0, 32 experts per step
  if (warp == 0) {
    int carry = 0;
    for (int base = 1; base <= E; base += 32) {
      const int idx = base + lane;
      int v = (idx <= E) ? blk_cum[idx] : 0;
#pragma unroll
      for (int off = 1; off < 32; off <<= 1) {
        const int n = __shfl_up_sync(0xffffffffu, v, off);
        if (lane >= off) v += n;
      }
      v += carry;
      if (idx <= E) blk_cum[idx] = v;
      carry = __shfl_sync(0xffffffffu, v, 31);
    }
  }
  __syncthreads();

  for (int e = tid; e <= E; e += kSortThreads) {
    if (mblk_cum) mblk_cum[e] = blk_cum[e];
    if (e < E && sorted_expert_ids)
      for (int b = blk_cum[e]; b < blk_cum[e + 1]; ++b) sorted_expert_ids[b] = e;
  }
  if (tid == 0 && num_post_pad) num_post_pad[0] = blk_cum[E] * block_m;
  if (tid == 0 && status_to_clear) status_to_clear[0] = 0;

  // pass 2: placement (same four-group prefetch, weights included)
  for (int r0 = r_begin; r0 < r_end; r0 += 32 * kUnroll) {
    int ev[kUnroll];
    float wv[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const int r = r0 + u * 32 + lane;
      ev[u] = (r < r_end) ? topk_ids[r] : -1;
      wv[u] = (r < r_end && sorted_weights) ? topk_weight[r] : 0.0f;
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      if (r0 + u * 32 >= r_end) break;               // warp-uniform
      const int r = r0 + u * 32 + lane;
      int e = ev[u];
      e = (e < 0 || e >= id_limit) ? -1 : e / id_div;
      const unsigned mask = __match_any_sync(0xffffffffu, e);
      if (e >= 0) {
        const int rank = __popc(mask & ((1u << lane) - 1u));
        const int pos = blk_cum[e] * block_m + my_cnt[e] + rank;
        sorted_token_ids[pos] = r / K;
        if (sorted_weights) sorted_weights[pos] = wv[u];
        if (sorted_rows) sorted_rows[pos] = r;
        if (inv_out) inv_out[r] = pos;
      } else if (inv_out && r < r_end) {
        inv_out[r] = -1;
      }
      __syncwarp();
      if (e >= 0 && lane == (__ffs(mask) - 1)) my_cnt[e] += __popc(mask);
      __syncwarp();
    }
  }
}

// ============================================================================= multi-CTA path
// For tens of thousands of pairs one SM's load/store unit is the limit (the scattered
// placement stores), so the same algorithm is spread over up to kSortMaxCtas CTAs in three
// launches: count (per-CTA histograms + pad fill), scan (one CTA: prefix over CTAs and over
// experts, block table), place (per-warp ranks inside each CTA on top of the CTA's base).
// The order inside an expert stays (CTA, warp, position): identical output to the one-CTA
// kernel.
struct SortRange {
  int T, R, r_begin, r_end;      // this warp's slice of the flat pair range
};

__device__ __forceinline__ SortRange sort_range(int T_max, const int32_t* num_tokens_dev, int K, int n_ctas,
                                                int cta, int warp) {
  SortRange s;
  s.T = num_tokens_dev ? min(T_max, max(0, *num_tokens_dev)) : T_max;
  s.R = s.T * K;
  // per-CTA chunk: a multiple of 1024 so every warp owns whole 32-wide groups
  const int cta_chunk = ((s.R + n_ctas - 1) / n_ctas + 1023) & ~1023;
  const int warp_chunk = cta_chunk / kSortWarps;
  s.r_begin = min(s.R, cta * cta_chunk + warp * warp_chunk);
  s.r_end = min(s.R, s.r_begin + warp_chunk);
  return s;
}

__device__ __forceinline__ void warp_histogram(const int32_t* __restrict__ topk_ids, int r_begin, int r_end,
                                               int id_limit, int id_div, int32_t* my_cnt, int lane) {
  constexpr int kUnroll = 4;
  for (int r0 = r_begin; r0 < r_end; r0 += 32 * kUnroll) {
    int ev[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const int r = r0 + u * 32 + lane;
      ev[u] = (r < r_end) ? topk_ids[r] : -1;
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      if (r0 + u * 32 >= r_end) break;               // warp-uniform
      int e = ev[u];
      e = (e < 0 || e >= id_limit) ? -1 : e / id_div;
      const unsigned mask = __match_any_sync(0xffffffffu, e);
      if (e >= 0 && lane == (__ffs(mask) - 1)) my_cnt[e] += __popc(mask);
      __syncwarp();
    }
  }
}

__global__ void __launch_bounds__(kSortThreads, 1)
sort_count_kernel(const int32_t* __restrict__ topk_ids, int T_max, const int32_t* __restrict__ num_tokens_dev,
                  int K, int E, int id_div, int block_m, int cap, int32_t* __restrict__ sorted_token_ids,
                  float* __restrict__ sorted_weights, int32_t* __restrict__ sorted_rows,
                  int32_t* __restrict__ sorted_expert_ids, int32_t* __restrict__ cnt_cta) {
  ptx::pdl_wait();
  ptx::pdl_release();
  extern __shared__ int32_t sm[];
  int32_t* cnt = sm;                                   // [kSortWarps][E]
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const SortRange sr = sort_range(T_max, num_tokens_dev, K, gridDim.x, blockIdx.x, warp);
  for (int i = tid; i < kSortWarps * E; i += kSortThreads) cnt[i] = 0;
  // pad fill, spread over the CTAs
  for (int i = blockIdx.x * kSortThreads + tid; i < cap; i += gridDim.x * kSortThreads) {
    sorted_token_ids[i] = T_max;
    if (sorted_weights) sorted_weights[i] = 0.0f;
    if (sorted_rows) sorted_rows[i] = -1;
    if (sorted_expert_ids && i < cap / block_m) sorted_expert_ids[i] = -1;
  }
  __syncthreads();
  warp_histogram(topk_ids, sr.r_begin, sr.r_end, E * id_div, id_div, cnt + warp * E, lane);
  __syncthreads();
  for (int e = tid; e < E; e += kSortThreads) {
    int run = 0;
    for (int w = 0; w < kSortWarps; ++w) run += cnt[w * E + e];
    cnt_cta[blockIdx.x * E + e] = run;
  }
}

__global__ void __launch_bounds__(kSortThreads, 1)
sort_scan_kernel(const int32_t* __restrict__ cnt_cta, int n_ctas, int E, int block_m,
                 int32_t* __restrict__ cta_base, int32_t* __restrict__ sorted_expert_ids,
                 int32_t* __restrict__ num_post_pad, int32_t* __restrict__ mblk_cum,
                 int32_t* __restrict__ status_to_clear) {
  ptx::pdl_wait();
  ptx::pdl_release();
  extern __shared__ int32_t sm[];
  int32_t* blk_cum = sm;                               // [E + 1]
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  for (int e = tid; e < E; e += kSortThreads) {
    int run = 0;
    for (int c = 0; c < n_ctas; ++c) {
      const int v = cnt_cta[c * E + e];
      cta_base[c * E + e] = run;                       // pairs of expert e in earlier CTAs
      run += v;
    }
    blk_cum[e + 1] = (run + block_m - 1) / block_m;
  }
  if (tid == 0) blk_cum[0] = 0;
  __syncthreads();
  if (warp == 0) {
    int carry = 0;
    for (int base = 1; base <= E; base += 32) {
      const int idx = base + lane;
      int v = (idx <= E) ? blk_cum[idx] : 0;
#pragma unroll
      for (int off = 1; off < 32; off <<= 1) {
        const int n = __shfl_up_sync(0xffffffffu, v, off);
        if (lane >= off) v += n;
      }
      v += carry;
      if (idx <= E) blk_cum[idx] = v;
      carry = __shfl_sync(0xffffffffu, v, 31);
    }
  }
  __syncthreads();
  for (int e = tid; e <= E; e += kSortThreads) {
    if (mblk_cum) mblk_cum[e] = blk_cum[e];
    if (e < E && sorted_expert_ids)
      for (int b = blk_cum[e]; b < blk_cum[e + 1]; ++b) sorted_expert_ids[b] = e;
  }
  if (tid == 0 && num_post_pad) num_post_pad[0] = blk_cum[E] * block_m;
  if (tid == 0 && status_to_clear) status_to_clear[0] = 0;
}

__global__ void __launch_bounds__(kSortThreads, 1)
sort_place_kernel(const int32_t* __restrict__ topk_ids, const float* __restrict__ topk_weight, int T_max,
                  const int32_t* __restrict__ num_tokens_dev, int K, int E, int id_div, int block_m,
                  const int32_t* __restrict__ cta_base, const int32_t* __restrict__ mblk_cum,
                  int32_t* __restrict__ sorted_token_ids, float* __restrict__ sorted_weights,
                  int32_t* __restrict__ sorted_rows, int32_t* __restrict__ inv_out) {
  ptx::pdl_wait();
  ptx::pdl_release();
  extern __shared__ int32_t sm[];
  int32_t* cnt = sm;                                   // [kSortWarps][E] counts -> running offsets
  int32_t* ebase = sm + kSortWarps * E;                // [E] first slot of expert e for this CTA
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const SortRange sr = sort_range(T_max, num_tokens_dev, K, gridDim.x, blockIdx.x, warp);
  const int id_limit = E * id_div;
  for (int i = tid; i < kSortWarps * E; i += kSortThreads) cnt[i] = 0;
  __syncthreads();
  int32_t* my_cnt = cnt + warp * E;
  warp_histogram(topk_ids, sr.r_begin, sr.r_end, id_limit, id_div, my_cnt, lane);
  __syncthreads();
  for (int e = tid; e < E; e += kSortThreads) {
    int run = 0;
    for (int w = 0; w < kSortWarps; ++w) {
      const int c = cnt[w * E + e];
      cnt[w * E + e] = run;
      run += c;
    }
    ebase[e] = mblk_cum[e] * block_m + cta_base[blockIdx.x * E + e];
  }
  __syncthreads();
  constexpr int kUnroll = 4;
  for (int r0 = sr.r_begin; r0 < sr.r_end; r0 += 32 * kUnroll) {
    int ev[kUnroll];
    float wv[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const int r = r0 + u * 32 + lane;
      ev[u] = (r < sr.r_end) ? topk_ids[r] : -1;
      wv[u] = (r < sr.r_end && sorted_weights) ? topk_weight[r] : 0.0f;
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      if (r0 + u * 32 >= sr.r_end) break;            // warp-uniform
      const int r = r0 + u * 32 + lane;
      int e = ev[u];
      e = (e < 0 || e >= id_limit) ? -1 : e / id_div;
      const unsigned mask = __match_any_sync(0xffffffffu, e);
      if (e >= 0) {
        const int rank = __popc(mask & ((1u << lane) - 1u));
        const int pos = ebase[e] + my_cnt[e] + rank;
        sorted_token_ids[pos] = r / K;
        if (sorted_weights) sorted_weights[pos] = wv[u];
        if (sorted_rows) sorted_rows[pos] = r;
        if (inv_out) inv_out[r] = pos;
      } else if (inv_out && r < sr.r_end) {
        inv_out[r] = -1;
      }
      __syncwarp();
      if (e >= 0 && lane == (__ffs(mask) - 1)) my_cnt[e] += __popc(mask);
      __syncwarp();
    }
  }
}

}  // namespace

cudaError_t launch_moe_sorting(const int32_t* topk_ids, const float* topk_weight, int T, int K,
                               int E, int block_m, int64_t cap, int32_t* sorted_token_ids,
                               float* sorted_weights, int32_t* sorted_rows,
                               int32_t* sorted_expert_ids, int32_t* num_post_pad,
                               int32_t* mblk_cum, int32_t* status_to_clear, cudaStream_t stream,
                               const int32_t* num_tokens_dev, int id_div, int32_t* inv_out,
                               int32_t* scratch) {
  const long long r_max = static_cast<long long>(T) * K;
  if (scratch != nullptr && mblk_cum != nullptr && r_max >= kSortMultiCtaMinPairs) {
    int n_ctas = static_cast<int>((r_max + 2047) / 2048);
    if (n_ctas > kSortMaxCtas) n_ctas = kSortMaxCtas;
    int32_t* cnt_cta = scratch;
    int32_t* cta_base = scratch + static_cast<size_t>(kSortMaxCtas) * E;
    const size_t smem_cnt = (static_cast<size_t>(kSortWarps) * E + E) * sizeof(int32_t);
    // opt in to large dynamic shared memory (E up to 1024) once per device: the attribute
    // belongs to the device the function is loaded on
    constexpr int kMaxDevices = 64;
    static bool configured[kMaxDevices] = {false};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= kMaxDevices || !configured[dev]) {
      cudaError_t e1 = cudaFuncSetAttribute(sort_count_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
      cudaError_t e2 = cudaFuncSetAttribute(sort_place_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
      if (e1 != cudaSuccess) return e1;
      if (e2 != cudaSuccess) return e2;
      if (dev >= 0 && dev < kMaxDevices) configured[dev] = true;
    }
    cudaError_t e = launch_pdl(sort_count_kernel, dim3(n_ctas), dim3(kSortThreads), smem_cnt, stream, topk_ids, T,
                               num_tokens_dev, K, E, id_div, block_m, static_cast<int>(cap), sorted_token_ids,
                               sorted_weights, sorted_rows, sorted_expert_ids, cnt_cta);
    if (e != cudaSuccess) return e;
    e = launch_pdl(sort_scan_kernel, dim3(1), dim3(kSortThreads), (static_cast<size_t>(E) + 1) * sizeof(int32_t),
                   stream, static_cast<const int32_t*>(cnt_cta), n_ctas, E, block_m, cta_base, sorted_expert_ids,
                   num_post_pad, mblk_cum, status_to_clear);
    if (e != cudaSuccess) return e;
    return launch_pdl(sort_place_kernel, dim3(n_ctas), dim3(kSortThreads), smem_cnt, stream, topk_ids, topk_weight,
                      T, num_tokens_dev, K, E, id_div, block_m, static_cast<const int32_t*>(cta_base),
                      static_cast<const int32_t*>(mblk_cum), sorted_token_ids, sorted_weights, sorted_rows, inv_out);
  }
  const size_t smem = (static_cast<size_t>(kSortWarps) * E + E + 1) * sizeof(int32_t);
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(moe_sorting_kernel,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         static_cast<int>(smem));
    if (e != cudaSuccess) return e;
  }
  return launch_pdl(moe_sorting_kernel, dim3(1), dim3(kSortThreads), smem, stream, topk_ids, topk_weight, T,
                    num_tokens_dev, K, E, id_div, block_m, static_cast<int>(cap), sorted_token_ids,
                    sorted_weights, sorted_rows, sorted_expert_ids, num_post_pad, mblk_cum, status_to_clear,
                    inv_out);
}

}  // namespace fmoe
