// Row-wise helper kernels of the fused-MoE operator (all HBM-bound, 16-byte vector access):
//   gather_rows  : activations -> sorted order (the A operand of the grouped GEMMs), with
//                  optional dynamic e4m3 quantisation per row or per 128-column group;
//                  the same kernel with identity indices quantises the intermediate.
//   combine      : out[t] = bf16( sum over k, ascending, of the weighted expert outputs ).
#include <cuda_bf16.h>
#include <cuda_fp8.h>

#include "internal.h"
#include "ptx.cuh"
#include "scales.cuh"

namespace fmoe {
namespace {

constexpr int kRowThreads = 128;

__device__ __forceinline__ float bf16_bits_to_f32(uint32_t bits16) {
  return __uint_as_float(bits16 << 16);
}

__device__ __forceinline__ void unpack8(const uint4& v, float (&f)[8]) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    f[2 * i] = bf16_bits_to_f32(w[i] & 0xffffu);
    f[2 * i + 1] = bf16_bits_to_f32(w[i] >> 16);
  }
}

__device__ __forceinline__ uint32_t e4m3_byte(float x) {
  return static_cast<uint32_t>(__nv_cvt_float_to_fp8(x, __NV_SATFINITE, __NV_E4M3));
}

// quantise 8 floats into 8 bytes: q = e4m3(v * inv_scale), inv_scale = 1/scale rounded once
__device__ __forceinline__ uint2 quant8(const float (&f)[8], float inv_scale) {
  uint32_t lo = 0, hi = 0;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    lo |= e4m3_byte(f[i] * inv_scale) << (8 * i);
    hi |= e4m3_byte(f[4 + i] * inv_scale) << (8 * i);
  }
  return make_uint2(lo, hi);
}

// One CTA per sorted slot.  kHeld: 16-byte vectors of the row one thread keeps in registers in
// the per-row mode (4 covers rows of up to 4096 elements with 128 threads); a smaller value
// means fewer registers, more resident CTAs and more bytes in flight for the common widths.
template <int kQuant, int kHeld = 16>
__global__ void __launch_bounds__(kRowThreads)
gather_rows_kernel(const uint4* __restrict__ src, int n_src, int cols,
                   const int32_t* __restrict__ row_ids, const int32_t* __restrict__ num_post_pad,
                   void* __restrict__ dst, void* __restrict__ scales_v,
                   const int32_t* __restrict__ live_ids, int skip_pad) {
  float* scales = reinterpret_cast<float*>(scales_v);
  ptx::pdl_wait();
  ptx::pdl_release();
  const int slot = blockIdx.x;
  if (num_post_pad != nullptr && slot >= *num_post_pad) return;
  // identity mode (quantising the intermediate): slots without a token are skipped outright
  if (live_ids != nullptr && live_ids[slot] < 0) return;
  const int row = row_ids ? row_ids[slot] : slot;
  const int nvec = cols >> 3;                       // 8 bf16 per 16-byte vector
  const bool pad = row < 0 || row >= n_src;
  // Inside the operator the rows of pad slots are never looked at again (every later kernel
  // skips the results of slots without a token), so they are not written: a quarter of the
  // traffic on fine-grained shapes.  The stand-alone pack helper keeps its zero rows.
  if (pad && skip_pad) return;
  const uint4* s = src + static_cast<size_t>(pad ? 0 : row) * nvec;

  if (kQuant == 0) {
    uint4* d = reinterpret_cast<uint4*>(dst) + static_cast<size_t>(slot) * nvec;
    for (int i = threadIdx.x; i < nvec; i += kRowThreads)
      d[i] = pad ? make_uint4(0, 0, 0, 0) : s[i];
    return;
  }

  uint2* d = reinterpret_cast<uint2*>(dst) + static_cast<size_t>(slot) * nvec;
  if (kQuant == 1) {
    // per-row scale: the row is read once into registers (up to kMaxVec vectors per thread,
    // i.e. rows of up to 16384 elements with 128 threads), reduced block-wide, then quantised from registers;
    // longer rows fall back to a second read.
    constexpr int kMaxVec = kHeld;
    __shared__ float warp_max[kRowThreads / 32];
    __shared__ float row_scale;
    const bool in_regs = nvec <= kMaxVec * kRowThreads;
    uint4 held[kMaxVec];
    float amax = 0.0f;
    if (!pad) {
#pragma unroll
      for (int j = 0; j < kMaxVec; ++j) {
        const int i = threadIdx.x + j * kRowThreads;
        if (in_regs && i < nvec) {
          held[j] = s[i];
          float f[8];
          unpack8(held[j], f);
#pragma unroll
          for (int e = 0; e < 8; ++e) amax = fmaxf(amax, fabsf(f[e]));
        }
      }
      if (!in_regs) {
        for (int i = threadIdx.x; i < nvec; i += kRowThreads) {
          float f[8];
          unpack8(s[i], f);
#pragma unroll
          for (int e = 0; e < 8; ++e) amax = fmaxf(amax, fabsf(f[e]));
        }
      }
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
    if ((threadIdx.x & 31) == 0) warp_max[threadIdx.x >> 5] = amax;
    __syncthreads();
    if (threadIdx.x == 0) {
      float m = 0.0f;
#pragma unroll
      for (int w = 0; w < kRowThreads / 32; ++w) m = fmaxf(m, warp_max[w]);
      const float sc = m > 0.0f ? m / 448.0f : 1.0f;
      row_scale = sc;
      scales[slot] = sc;
    }
    __syncthreads();
    const float sc = 1.0f / row_scale;
    if (pad) {
      for (int i = threadIdx.x; i < nvec; i += kRowThreads) d[i] = make_uint2(0, 0);
    } else if (in_regs) {
#pragma unroll
      for (int j = 0; j < kMaxVec; ++j) {
        const int i = threadIdx.x + j * kRowThreads;
        if (i < nvec) {
          float f[8];
          unpack8(held[j], f);
          d[i] = quant8(f, sc);
        }
      }
    } else {
      for (int i = threadIdx.x; i < nvec; i += kRowThreads) {
        float f[8];
        unpack8(s[i], f);
        d[i] = quant8(f, sc);
      }
    }
  } else {
    // one scale per 128 columns = 16 vectors = a 16-lane group.  Up to kGroupVec vectors per
    // thread are loaded before any is processed so the loads overlap.
    constexpr int kGroupVec = 8;
    const int ngroups = cols >> 7;
    for (int base = 0; base < nvec; base += kRowThreads * kGroupVec) {   // warp-uniform trip count
      uint4 held[kGroupVec];
#pragma unroll
      for (int j = 0; j < kGroupVec; ++j) {
        const int i = base + j * kRowThreads + threadIdx.x;
        held[j] = (i < nvec && !pad) ? s[i] : make_uint4(0, 0, 0, 0);
      }
#pragma unroll
      for (int j = 0; j < kGroupVec; ++j) {
        const int i = base + j * kRowThreads + threadIdx.x;      // nvec is a multiple of 16
        float f[8];
        unpack8(held[j], f);
        float amax = 0.0f;
#pragma unroll
        for (int e = 0; e < 8; ++e) amax = fmaxf(amax, fabsf(f[e]));
#pragma unroll
        for (int off = 8; off > 0; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
        uint32_t sbyte;
        const float sc = group_scale<kQuant == 3>(amax, sbyte);
        if (i < nvec) {
          if ((i & 15) == 0) {
            if (kQuant == 3)   // one UE8M0 byte per row and K group
              reinterpret_cast<uint8_t*>(scales_v)[static_cast<size_t>(slot) * scale_pitch(ngroups) + (i >> 4)] =
                  static_cast<uint8_t>(sbyte);
            else
              scales[static_cast<size_t>(slot) * ngroups + (i >> 4)] = sc;
          }
          d[i] = quant8(f, 1.0f / sc);
        }
      }
    }
  }
}

template <bool kBf16Slots>
__global__ void __launch_bounds__(kRowThreads)
combine_kernel(const void* __restrict__ slots_v, const int32_t* __restrict__ topk_ids, int K, int E,
               int H, void* __restrict__ out_v, const int32_t* __restrict__ num_tokens_dev) {
  ptx::pdl_wait();
  ptx::pdl_release();
  const int t = blockIdx.x;
  if (num_tokens_dev && t >= *num_tokens_dev) return;   // rows past the device-side count
  // grid.y spreads a row's vectors over several CTAs, so a thread has few dependent loads
  const int i0 = blockIdx.y * kRowThreads + threadIdx.x;
  const int istep = gridDim.y * kRowThreads;
  if (kBf16Slots) {
    // bf16 partial rows: 8 elements (16 bytes) per thread and term
    const int nvec = H >> 3;
    const uint4* slots = reinterpret_cast<const uint4*>(slots_v);
    uint4* out = reinterpret_cast<uint4*>(out_v);
    for (int i = i0; i < nvec; i += istep) {
      float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
      for (int k = 0; k < K; ++k) {
        const int e = topk_ids[t * K + k];
        if (e < 0 || e >= E) continue;
        float f[8];
        unpack8(slots[(static_cast<size_t>(t) * K + k) * nvec + i], f);
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] += f[j];
      }
      uint32_t w[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        __nv_bfloat162 v = __floats2bfloat162_rn(acc[2 * j], acc[2 * j + 1]);
        w[j] = *reinterpret_cast<uint32_t*>(&v);
      }
      out[static_cast<size_t>(t) * nvec + i] = make_uint4(w[0], w[1], w[2], w[3]);
    }
    return;
  }
  const int nvec = H >> 2;
  const float4* slots = reinterpret_cast<const float4*>(slots_v);
  uint2* out = reinterpret_cast<uint2*>(out_v);
  for (int i = i0; i < nvec; i += istep) {
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int k = 0; k < K; ++k) {
      const int e = topk_ids[t * K + k];
      if (e < 0 || e >= E) continue;
      const float4 v = slots[(static_cast<size_t>(t) * K + k) * nvec + i];
      acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    __nv_bfloat162 lo = __floats2bfloat162_rn(acc.x, acc.y);
    __nv_bfloat162 hi = __floats2bfloat162_rn(acc.z, acc.w);
    out[static_cast<size_t>(t) * nvec + i] =
        make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
  }
}

// Rows that are already quantised (one pass over the T token rows) -> sorted order: each routed
// pair copies its token's e4m3 row and scale(s).  With K experts per token this moves K e4m3 rows
// instead of quantising the same bf16 row K times.  Pad slots are left unwritten.
//   kQuant 1: scales f32 [rows]; 2: f32 [rows, cols/128]; 3: UE8M0 bytes [rows, pitch].
template <int kQuant>
__global__ void __launch_bounds__(kRowThreads)
gather_quantised_kernel(const uint4* __restrict__ src, const void* __restrict__ src_scale, int n_src, int cols,
                        const int32_t* __restrict__ row_ids, const int32_t* __restrict__ num_post_pad,
                        uint4* __restrict__ dst, void* __restrict__ dst_scale) {
  ptx::pdl_wait();
  ptx::pdl_release();
  const int slot = blockIdx.x;
  if (slot >= *num_post_pad) return;
  const int row = row_ids[slot];
  if (row < 0 || row >= n_src) return;
  const int nvec = cols >> 4;                       // 16 e4m3 per 16-byte vector
  const uint4* s = src + static_cast<size_t>(row) * nvec;
  uint4* d = dst + static_cast<size_t>(slot) * nvec;
  for (int i = threadIdx.x; i < nvec; i += kRowThreads) d[i] = s[i];
  if (kQuant == 1) {
    if (threadIdx.x == 0) reinterpret_cast<float*>(dst_scale)[slot] = reinterpret_cast<const float*>(src_scale)[row];
  } else {
    // 32-bit words per row: cols/128 floats, or pitch/4 words of packed UE8M0 bytes
    const int words = kQuant == 2 ? (cols >> 7) : (scale_pitch(cols >> 7) >> 2);
    const uint32_t* ss = reinterpret_cast<const uint32_t*>(src_scale) + static_cast<size_t>(row) * words;
    uint32_t* ds = reinterpret_cast<uint32_t*>(dst_scale) + static_cast<size_t>(slot) * words;
    for (int i = threadIdx.x; i < words; i += kRowThreads) ds[i] = ss[i];
  }
}

// ----------------------------------------------------------------------------- decode prologue
// moe_sorting + gather (+ per-token quantisation) in one launch for decode-sized batches: at
// most kProloguePairs routed pairs, so every expert that is hit owns exactly one row block.
// One CTA per routed pair: each CTA reads all the ids (a few hundred bytes), works out the slot of
// its own pair with block-wide counts -- bit-identical to the moe_sorting kernels -- and moves its
// row; CTA 0 also writes the sorted arrays, the block table and the counters.  Pad slots of the
// activation matrix are left untouched: their rows of every later result are never stored.
constexpr int kProloguePairs = 128;

template <int kQuant>
__global__ void __launch_bounds__(kRowThreads)
decode_prologue_kernel(const int32_t* __restrict__ topk_ids, const float* __restrict__ topk_weight, int T_max,
                       const int32_t* __restrict__ num_tokens_dev, int K, int E, int cap, const uint4* __restrict__ x,
                       int H, int32_t* __restrict__ sorted_token_ids, float* __restrict__ sorted_weights,
                       int32_t* __restrict__ sorted_rows, int32_t* __restrict__ sorted_expert_ids,
                       int32_t* __restrict__ num_post_pad, int32_t* __restrict__ mblk_cum,
                       int32_t* __restrict__ status_to_clear, void* __restrict__ a_sorted, float* __restrict__ a_scale) {
  ptx::pdl_wait();
  ptx::pdl_release();
  __shared__ int32_t ids_s[kProloguePairs];
  __shared__ int32_t slot_s[kProloguePairs];
  __shared__ int32_t first_s[kProloguePairs];
  __shared__ float warp_max[kRowThreads / 32];
  __shared__ float row_scale;
  const int tid = threadIdx.x;
  const int T = num_tokens_dev ? min(T_max, max(0, *num_tokens_dev)) : T_max;
  const int R = T * K;                               // <= kProloguePairs (checked by the launcher)
  int my_e = -1;
  if (tid < R) {
    const int e = topk_ids[tid];
    my_e = (e >= 0 && e < E) ? e : -1;
  }
  if (tid < kProloguePairs) ids_s[tid] = my_e;
  __syncthreads();
  // first_s[j]: pair j is the first pair of its expert.  The slot of pair `tid` is
  // (experts below mine that are hit) * 128 + (earlier pairs of my expert).
  int rank = 0;
  if (tid < kProloguePairs) {
    bool first = my_e >= 0;
    if (my_e >= 0)
      for (int j = 0; j < tid; ++j) {
        const bool same = ids_s[j] == my_e;
        rank += same;
        first = first && !same;
      }
    first_s[tid] = first ? 1 : 0;
  }
  __syncthreads();
  if (tid < R) {
    int blocks_before = 0;
    if (my_e >= 0)
      for (int j = 0; j < R; ++j) blocks_before += (first_s[j] && ids_s[j] < my_e);
    slot_s[tid] = my_e >= 0 ? blocks_before * 128 + rank : -1;
  }
  __syncthreads();

  if (blockIdx.x == 0) {
    // sorted arrays, block table and counters (what the moe_sorting kernel writes)
    for (int i = tid; i < cap; i += kRowThreads) {
      sorted_token_ids[i] = T_max;
      sorted_weights[i] = 0.0f;
      sorted_rows[i] = -1;
    }
    for (int i = tid; i < cap / 128; i += kRowThreads) sorted_expert_ids[i] = -1;
    __syncthreads();
    if (tid < R && slot_s[tid] >= 0) {
      const int sl = slot_s[tid];
      sorted_token_ids[sl] = tid / K;
      sorted_weights[sl] = topk_weight[tid];
      sorted_rows[sl] = tid;
      if ((sl & 127) == 0) sorted_expert_ids[sl >> 7] = my_e;
    }
    // cumulative blocks per expert: experts that are hit own one block each
    for (int e = tid; e <= E; e += kRowThreads) {
      int below = 0;                                 // distinct hit experts with id < e
      for (int j = 0; j < R; ++j) below += (first_s[j] && ids_s[j] < e);
      mblk_cum[e] = below;
      if (e == E) num_post_pad[0] = below * 128;
    }
    if (tid == 0 && status_to_clear) status_to_clear[0] = 0;
  }

  // this CTA's row
  const int pair = blockIdx.x;
  if (pair >= R) return;
  const int slot = slot_s[pair];
  if (slot < 0) return;
  const int nvec = H >> 3;
  const uint4* src = x + static_cast<size_t>(pair / K) * nvec;
  if (kQuant == 0) {
    uint4* d = reinterpret_cast<uint4*>(a_sorted) + static_cast<size_t>(slot) * nvec;
    for (int i = tid; i < nvec; i += kRowThreads) d[i] = src[i];
    return;
  }
  float amax = 0.0f;
  for (int i = tid; i < nvec; i += kRowThreads) {
    float f[8];
    unpack8(src[i], f);
#pragma unroll
    for (int e = 0; e < 8; ++e) amax = fmaxf(amax, fabsf(f[e]));
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
  if ((tid & 31) == 0) warp_max[tid >> 5] = amax;
  __syncthreads();
  if (tid == 0) {
    float m = 0.0f;
#pragma unroll
    for (int w = 0; w < kRowThreads / 32; ++w) m = fmaxf(m, warp_max[w]);
    const float sc = m > 0.0f ? m / 448.0f : 1.0f;
    row_scale = sc;
    a_scale[slot] = sc;
  }
  __syncthreads();
  const float inv = 1.0f / row_scale;
  uint2* d = reinterpret_cast<uint2*>(a_sorted) + static_cast<size_t>(slot) * nvec;
  for (int i = tid; i < nvec; i += kRowThreads) {
    float f[8];
    unpack8(src[i], f);                               // second read of the row comes from L1/L2
    d[i] = quant8(f, inv);
  }
}

// Expert-parallel combine: bf16 partial rows picked through an index, f32 sum in k order.
__global__ void __launch_bounds__(kRowThreads)
combine_rows_kernel(const uint4* __restrict__ rows, const int32_t* __restrict__ index, int K, int H,
                    uint4* __restrict__ out) {
  const int t = blockIdx.x;
  const int nvec = H >> 3;
  for (int i = threadIdx.x; i < nvec; i += kRowThreads) {
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int k = 0; k < K; ++k) {
      const int r = index[t * K + k];
      if (r < 0) continue;
      float f[8];
      unpack8(rows[static_cast<size_t>(r) * nvec + i], f);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] += f[j];
    }
    uint32_t w[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      __nv_bfloat162 v = __floats2bfloat162_rn(acc[2 * j], acc[2 * j + 1]);
      w[j] = *reinterpret_cast<uint32_t*>(&v);
    }
    out[static_cast<size_t>(t) * nvec + i] = make_uint4(w[0], w[1], w[2], w[3]);
  }
}

}  // namespace

cudaError_t launch_combine_rows(const void* rows, const int32_t* index, int T, int K, int H,
                                void* out, cudaStream_t stream) {
  combine_rows_kernel<<<T, kRowThreads, 0, stream>>>(reinterpret_cast<const uint4*>(rows), index, K, H,
                                                     reinterpret_cast<uint4*>(out));
  return cudaGetLastError();
}

cudaError_t launch_gather_rows(const void* src, int n_src, int cols, const int32_t* row_ids,
                               const int32_t* num_post_pad, int64_t cap, int quant, void* dst,
                               void* scales, cudaStream_t stream, const int32_t* live_ids, bool skip_pad) {
  const dim3 grid(static_cast<unsigned>(cap));
  const uint4* s = reinterpret_cast<const uint4*>(src);
  const int sp = skip_pad ? 1 : 0;
  if (quant == 0)
    return launch_pdl(gather_rows_kernel<0>, grid, dim3(kRowThreads), 0, stream, s, n_src, cols, row_ids, num_post_pad, dst, scales, live_ids, sp);
  else if (quant == 1) {
    const int nvec = cols >> 3;
    if (nvec <= 4 * kRowThreads)
      return launch_pdl(gather_rows_kernel<1, 4>, grid, dim3(kRowThreads), 0, stream, s, n_src, cols, row_ids, num_post_pad, dst, scales, live_ids, sp);
    if (nvec <= 8 * kRowThreads)
      return launch_pdl(gather_rows_kernel<1, 8>, grid, dim3(kRowThreads), 0, stream, s, n_src, cols, row_ids, num_post_pad, dst, scales, live_ids, sp);
    return launch_pdl(gather_rows_kernel<1>, grid, dim3(kRowThreads), 0, stream, s, n_src, cols, row_ids, num_post_pad, dst, scales, live_ids, sp);
  }
  else if (quant == 2)
    return launch_pdl(gather_rows_kernel<2>, grid, dim3(kRowThreads), 0, stream, s, n_src, cols, row_ids, num_post_pad, dst, scales, live_ids, sp);
  else
    return launch_pdl(gather_rows_kernel<3>, grid, dim3(kRowThreads), 0, stream, s, n_src, cols, row_ids, num_post_pad, dst, scales, live_ids, sp);
}

cudaError_t launch_gather_quantised(const void* src, const void* src_scale, int n_src, int cols,
                                    const int32_t* row_ids, const int32_t* num_post_pad, int64_t cap, int quant,
                                    void* dst, void* dst_scale, cudaStream_t stream) {
  const dim3 grid(static_cast<unsigned>(cap));
  const uint4* s = reinterpret_cast<const uint4*>(src);
  uint4* d = reinterpret_cast<uint4*>(dst);
  if (quant == 1)
    return launch_pdl(gather_quantised_kernel<1>, grid, dim3(kRowThreads), 0, stream, s, src_scale, n_src, cols, row_ids, num_post_pad, d, dst_scale);
  if (quant == 2)
    return launch_pdl(gather_quantised_kernel<2>, grid, dim3(kRowThreads), 0, stream, s, src_scale, n_src, cols, row_ids, num_post_pad, d, dst_scale);
  return launch_pdl(gather_quantised_kernel<3>, grid, dim3(kRowThreads), 0, stream, s, src_scale, n_src, cols, row_ids, num_post_pad, d, dst_scale);
}

bool decode_prologue_applies(int T, int K, int quant) {
  return static_cast<long long>(T) * K <= kProloguePairs && (quant == 0 || quant == 1);
}

cudaError_t launch_decode_prologue(const int32_t* topk_ids, const float* topk_weight, int T, int K, int E, int64_t cap,
                                   const void* x, int H, int quant, int32_t* sorted_token_ids, float* sorted_weights,
                                   int32_t* sorted_rows, int32_t* sorted_expert_ids, int32_t* num_post_pad,
                                   int32_t* mblk_cum, int32_t* status_to_clear, void* a_sorted, float* a_scale,
                                   cudaStream_t stream, const int32_t* num_tokens_dev) {
  const dim3 grid(static_cast<unsigned>(T * K > 0 ? T * K : 1));
  const uint4* xs = reinterpret_cast<const uint4*>(x);
  if (quant == 0)
    return launch_pdl(decode_prologue_kernel<0>, grid, dim3(kRowThreads), 0, stream, topk_ids, topk_weight, T,
                      num_tokens_dev, K, E, static_cast<int>(cap), xs, H, sorted_token_ids, sorted_weights, sorted_rows,
                      sorted_expert_ids, num_post_pad, mblk_cum, status_to_clear, a_sorted, a_scale);
  return launch_pdl(decode_prologue_kernel<1>, grid, dim3(kRowThreads), 0, stream, topk_ids, topk_weight, T,
                    num_tokens_dev, K, E, static_cast<int>(cap), xs, H, sorted_token_ids, sorted_weights, sorted_rows,
                    sorted_expert_ids, num_post_pad, mblk_cum, status_to_clear, a_sorted, a_scale);
}

cudaError_t launch_combine(const void* slots, bool slots_bf16, const int32_t* topk_ids, int T, int K, int E,
                           int H, void* out, cudaStream_t stream, const int32_t* num_tokens_dev) {
  // few tokens: spread each row over several CTAs so the whole GPU takes part
  const int nvec = slots_bf16 ? H >> 3 : H >> 2;
  int gy = 1;
  if (T < 1024) {
    gy = (nvec + kRowThreads - 1) / kRowThreads;
    if (gy > 16) gy = 16;
  }
  if (slots_bf16)
    return launch_pdl(combine_kernel<true>, dim3(T, gy), dim3(kRowThreads), 0, stream, slots, topk_ids, K, E, H, out,
                      num_tokens_dev);
  return launch_pdl(combine_kernel<false>, dim3(T, gy), dim3(kRowThreads), 0, stream, slots, topk_ids, K, E, H, out,
                    num_tokens_dev);
}

}  // namespace fmoe
