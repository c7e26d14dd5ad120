// Expert-parallel dispatch / return over peer memory (NVLink P2P stores), one process per
// GPU.  Every rank owns one "symmetric" buffer with the same layout; peer_base[r] is the
// address of rank r's buffer as mapped into this process.  Nothing here synchronises with
// the host: counts, offsets and row counts stay on the device, and ranks meet at flag
// barriers whose spins are bounded.
//
//   plan      : bucket the routed pairs by owner rank (the moe_sorting kernel with
//               id / experts_per_rank as the bucket) -> send order, inverse index, counts
//   publish   : write my row of the rank x rank count matrix into every rank's copy
//   barrier   : epoch flags, release/acquire at system scope
//   dispatch  : one CTA per send slot: token row + (local expert, weight, source) to the
//               owner's receive arrays at  sum(counts of lower ranks) + index in my group
//   return    : one CTA per received row: the expert output back to the source's slot
#include <cuda_runtime.h>

#include "../../include/fused_moe_c.h"
#include "internal.h"
#include "plan.hpp"

namespace fmoe {
namespace {

constexpr int kEpThreads = 256;
constexpr int kMaxRanks = 64;

template <typename T>
__device__ __forceinline__ T* peer_ptr(const uint64_t* peer_base, int rank, uint64_t off) {
  return reinterpret_cast<T*>(peer_base[rank] + off);
}

__global__ void ep_publish_kernel(const int32_t* __restrict__ cum, const uint64_t* __restrict__ peer_base,
                                  uint64_t matrix_off, int me, int G) {
  // thread (p, d): rank p's copy of matrix[me][d] = rows I send to rank d
  for (int i = threadIdx.x; i < G * G; i += blockDim.x) {
    const int p = i / G, d = i % G;
    peer_ptr<int32_t>(peer_base, p, matrix_off)[me * G + d] = cum[d + 1] - cum[d];
  }
}

__global__ void ep_barrier_kernel(const uint64_t* __restrict__ peer_base, uint64_t flags_off, int me, int G,
                                  int epoch, int32_t* __restrict__ epoch_counter,
                                  int32_t* __restrict__ status, long long limit_cycles) {
  const int p = threadIdx.x;
  if (epoch_counter != nullptr) {
    // the epoch lives on the device: every launch (or graph replay) of this kernel advances it
    __shared__ int32_t next;
    if (threadIdx.x == 0) next = ++(*epoch_counter);
    __syncthreads();
    epoch = next;
  }
  if (p >= G) return;
  __threadfence_system();   // everything this rank wrote before the barrier is visible first
  volatile int32_t* theirs = peer_ptr<int32_t>(peer_base, p, flags_off) + me;
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(theirs), "r"(epoch) : "memory");
  const int32_t* mine = peer_ptr<int32_t>(peer_base, me, flags_off) + p;
  const long long t0 = clock64();
  int32_t v;
  for (;;) {
    asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(mine) : "memory");
    if (v >= epoch) break;
    if (clock64() - t0 > limit_cycles) {   // a rank never arrived: report, do not hang
      atomicExch(status, 0x300 | p);
      break;
    }
    __nanosleep(64);
  }
}

__global__ void __launch_bounds__(kEpThreads)
ep_dispatch_kernel(const uint4* __restrict__ x, const int32_t* __restrict__ topk_ids,
                   const float* __restrict__ topk_w, int K, int H, int e_local,
                   const int32_t* __restrict__ order, const int32_t* __restrict__ cum,
                   const uint64_t* __restrict__ peer_base, fmoe_ep_layout_c lay, int me, int G,
                   int32_t* __restrict__ n_recv_dev) {
  const int slot = blockIdx.x;
  const int32_t* matrix = peer_ptr<int32_t>(peer_base, me, lay.matrix);
  if (slot == 0 && threadIdx.x == 0) {
    int n = 0;
    for (int s = 0; s < G; ++s) n += matrix[s * G + me];
    *n_recv_dev = n;
  }
  if (slot >= cum[G]) return;
  int d = 0;
  while (d + 1 < G && slot >= cum[d + 1]) ++d;
  int base = 0;
  for (int s = 0; s < me; ++s) base += matrix[s * G + d];
  const int64_t dst = base + (slot - cum[d]);
  if (dst >= lay.recv_cap) return;   // cannot happen with recv_cap >= all routed pairs
  const int r = order[slot];
  const int t = r / K;
  const int nvec = H >> 3;
  const uint4* src = x + static_cast<size_t>(t) * nvec;
  uint4* rows = peer_ptr<uint4>(peer_base, d, lay.rows) + static_cast<size_t>(dst) * nvec;
  for (int i = threadIdx.x; i < nvec; i += kEpThreads) rows[i] = src[i];
  if (threadIdx.x == 0) {
    peer_ptr<int32_t>(peer_base, d, lay.ids)[dst] = topk_ids[r] % e_local;
    peer_ptr<float>(peer_base, d, lay.weights)[dst] = topk_w[r];
    peer_ptr<int2>(peer_base, d, lay.src)[dst] = make_int2(me, slot);
  }
}

__global__ void __launch_bounds__(kEpThreads)
ep_return_kernel(const uint4* __restrict__ out_rows, int H, const int32_t* __restrict__ n_recv_dev,
                 const uint64_t* __restrict__ peer_base, fmoe_ep_layout_c lay, int me, int G) {
  const int i = blockIdx.x;
  if (i >= *n_recv_dev) return;
  const int2 s = peer_ptr<int2>(peer_base, me, lay.src)[i];
  if (s.x < 0 || s.x >= G || s.y < 0 || s.y >= lay.send_cap) return;   // never follow a bad return address
  const int nvec = H >> 3;
  const uint4* src = out_rows + static_cast<size_t>(i) * nvec;
  uint4* dst = peer_ptr<uint4>(peer_base, s.x, lay.back) + static_cast<size_t>(s.y) * nvec;
  for (int v = threadIdx.x; v < nvec; v += kEpThreads) dst[v] = src[v];
}

}  // namespace

static int launch_status(const char* what) {
  const cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? FMOE_OK : fail(FMOE_ERR_CUDA, "%s launch failed: %s", what, cudaGetErrorString(e));
}
}  // namespace fmoe

extern "C" {

int fmoe_ep_plan(const int32_t* topk_ids, int32_t T, int32_t K, int32_t experts_per_rank, int32_t G,
                 int32_t* order, int32_t* inv_index, int32_t* cum, int32_t* scratch_tokens, void* stream) {
  if (!topk_ids || !order || !inv_index || !cum || !scratch_tokens)
    return fmoe::fail(FMOE_ERR_INVALID_ARG, "fmoe_ep_plan: topk_ids, order, inv_index, cum and scratch_tokens are required");
  if (T <= 0 || K <= 0 || experts_per_rank <= 0 || G <= 0 || G > fmoe::kMaxRanks)
    return fmoe::fail(FMOE_ERR_INVALID_ARG, "fmoe_ep_plan: bad dimensions (T=%d K=%d experts_per_rank=%d G=%d)", T, K,
                      experts_per_rank, G);
  // block size 1: no padding, so the cumulative block counts are the cumulative row counts
  cudaError_t e = fmoe::launch_moe_sorting(topk_ids, nullptr, T, K, G, 1, static_cast<int64_t>(T) * K,
                                           scratch_tokens, nullptr, order, nullptr, nullptr, cum, nullptr,
                                           static_cast<cudaStream_t>(stream), nullptr, experts_per_rank,
                                           inv_index);
  return e == cudaSuccess ? FMOE_OK : fmoe::fail(FMOE_ERR_CUDA, "fmoe_ep_plan: %s", cudaGetErrorString(e));
}

int fmoe_ep_publish(const int32_t* cum, const uint64_t* peer_base, const fmoe_ep_layout_c* lay, int32_t me,
                    int32_t G, void* stream) {
  if (!cum || !peer_base || !lay || G <= 0 || G > fmoe::kMaxRanks || me < 0 || me >= G)
    return fmoe::fail(FMOE_ERR_INVALID_ARG, "fmoe_ep_publish: null pointer or rank %d / world %d out of range", me, G);
  fmoe::ep_publish_kernel<<<1, 64, 0, static_cast<cudaStream_t>(stream)>>>(cum, peer_base, lay->matrix, me, G);
  return fmoe::launch_status("expert-parallel kernel");
}

int fmoe_ep_barrier(const uint64_t* peer_base, const fmoe_ep_layout_c* lay, int32_t me, int32_t G,
                    int32_t epoch, int32_t* epoch_counter, int32_t* status, int32_t timeout_ms, void* stream) {
  if (!peer_base || !lay || !status || G <= 0 || G > fmoe::kMaxRanks || me < 0 || me >= G || timeout_ms < 0)
    return fmoe::fail(FMOE_ERR_INVALID_ARG, "fmoe_ep_barrier: null pointer, negative timeout, or rank %d / world %d out of range", me, G);
  // clock64 ticks at the SM clock (<= ~2 GHz): 2e6 cycles per millisecond is an upper bound
  const long long limit = timeout_ms > 0 ? 2000000LL * timeout_ms : 8000000000LL;   // default: about four seconds
  fmoe::ep_barrier_kernel<<<1, 64, 0, static_cast<cudaStream_t>(stream)>>>(peer_base, lay->flags, me, G, epoch,
                                                                          epoch_counter, status, limit);
  return fmoe::launch_status("expert-parallel kernel");
}

int fmoe_ep_dispatch(const void* x, const int32_t* topk_ids, const float* topk_weight, int32_t T, int32_t K,
                     int32_t H, int32_t experts_per_rank, const int32_t* order, const int32_t* cum,
                     const uint64_t* peer_base, const fmoe_ep_layout_c* lay, int32_t me, int32_t G,
                     int32_t* n_recv_dev, void* stream) {
  if (!x || !topk_ids || !topk_weight || !order || !cum || !peer_base || !lay || !n_recv_dev)
    return fmoe::fail(FMOE_ERR_INVALID_ARG, "fmoe_ep_dispatch: a required pointer is null");
  if (G <= 0 || G > fmoe::kMaxRanks || me < 0 || me >= G)
    return fmoe::fail(FMOE_ERR_INVALID_ARG, "fmoe_ep_dispatch: rank %d / world %d out of range", me, G);
  if (H <= 0 || H % 8 || T <= 0 || K <= 0)
    return fmoe::fail(FMOE_ERR_UNSUPPORTED, "fmoe_ep_dispatch: H must be a positive multiple of 8 and T, K positive");
  fmoe::ep_dispatch_kernel<<<T * K, fmoe::kEpThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const uint4*>(x), topk_ids, topk_weight, K, H, experts_per_rank, order, cum, peer_base,
      *lay, me, G, n_recv_dev);
  return fmoe::launch_status("expert-parallel kernel");
}

int fmoe_ep_return(const void* out_rows, int32_t H, const int32_t* n_recv_dev, const uint64_t* peer_base,
                   const fmoe_ep_layout_c* lay, int32_t me, int32_t G, void* stream) {
  if (!out_rows || !n_recv_dev || !peer_base || !lay || G <= 0 || G > fmoe::kMaxRanks || me < 0 || me >= G)
    return fmoe::fail(FMOE_ERR_INVALID_ARG, "fmoe_ep_return: null pointer or rank %d / world %d out of range", me, G);
  if (lay->recv_cap <= 0) return FMOE_OK;
  fmoe::ep_return_kernel<<<static_cast<unsigned>(lay->recv_cap), fmoe::kEpThreads, 0,
                           static_cast<cudaStream_t>(stream)>>>(reinterpret_cast<const uint4*>(out_rows), H,
                                                                 n_recv_dev, peer_base, *lay, me, G);
  return fmoe::launch_status("expert-parallel kernel");
}

}  // extern "C"
