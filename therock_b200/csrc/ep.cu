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
#include <cuda_bf16.h>
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
  // the release store orders everything this rank wrote before the barrier (earlier kernels on the
  // stream included: the release is cumulative) before the flag
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


// ============================================================================= fused step
// Three kernels around the local operator: send (plan + publish + wait + dispatch + signal),
// recv_ready (wait + return-address table) and wait_combine (wait + ordered sum).

constexpr int kSendThreads = 256;
constexpr int kSendMaxRanks = 16;
constexpr int kSendMaxChunk = 2048;       // routed pairs one CTA of the send kernel handles
constexpr int kSendPairsPerCta = 8;       // target: enough CTAs to keep the links busy

__device__ __forceinline__ int ld_acquire_sys(const int32_t* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(int32_t* p, int v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
// Release fence at system scope, the acquire/release form (not the sequentially consistent
// membar.sys of __threadfence_system()).
__device__ __forceinline__ void fence_acq_rel_sys() { asm volatile("fence.acq_rel.sys;" ::: "memory"); }
// After one system-scope fence: fence + relaxed store is a release, without a fence per flag.
__device__ __forceinline__ void st_relaxed_sys(int32_t* p, int v) {
  asm volatile("st.relaxed.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_acquire_gpu(const int32_t* p) {
  int v;
  asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_gpu(int32_t* p, int v) {
  asm volatile("st.release.gpu.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
// All CTAs of a kernel wait until flags[p] >= epoch for every rank p.  Only the first two CTAs
// poll the flags the peers write (system scope); the one that sees them complete publishes the
// epoch in a local word the other CTAs poll at device scope with a growing back-off, so a
// thousand waiting CTAs do not hammer one line of memory with system-scope loads while copies
// and peer stores are in flight.  Gives up after `limit` cycles and reports the missing rank.
// Layout of the step's scratch words (int32): [0] grid barrier of the send kernel, [1] its
// finished CTAs, [2] / [3] / [4] the local "complete" words of the three waits, [5] finished CTAs
// of wait_combine, [8 ...] per-CTA counts of the send kernel.
__device__ __forceinline__ void wait_flags(const int32_t* flags, int32_t* ready, int G, int epoch, long long limit,
                                           int32_t* status) {
  if (threadIdx.x == 0) {
    const long long t0 = clock64();
    unsigned backoff = 32;
    for (;;) {
      if (ld_acquire_gpu(ready) >= epoch) break;
      if (blockIdx.x < 2) {
        int missing = -1;
        for (int p = 0; p < G; ++p)
          if (ld_acquire_sys(flags + p) < epoch) { missing = p; break; }
        if (missing < 0) {
          st_release_gpu(ready, epoch);
          break;
        }
        if (clock64() - t0 > limit) {
          atomicExch(status, 0x300 | missing);
          st_release_gpu(ready, epoch);          // let the other CTAs go on too: the step is lost anyway
          break;
        }
      } else if (clock64() - t0 > 2 * limit) {   // the polling CTAs never reported: do not wait for ever
        atomicExch(status, 0x330);
        break;
      }
      __nanosleep(backoff);
      if (backoff < 1024) backoff <<= 1;
    }
  }
  __syncthreads();
}

struct EpSendParams {
  const uint4* x;            // [T] rows of row_vecs 16-byte vectors
  const uint32_t* x_scale;   // [T] rows of scale_words 32-bit words, or nullptr
  int row_vecs, scale_words;
  const int32_t* topk_ids;
  const float* topk_w;
  int T, K, e_local;
  const uint64_t* peer_base;
  fmoe_ep_layout_c lay;
  int me, G;
  int32_t* cta_counts;     // [grid][G]
  int32_t* sync;           // [0] grid barrier, [1] finished CTAs
  const int32_t* epoch;
  int32_t* n_recv_dev;
  int32_t* status;
  long long limit;
};

__global__ void __launch_bounds__(kSendThreads)
ep_send_kernel(const EpSendParams p) {
  __shared__ int32_t tcnt[kSendThreads][kSendMaxRanks];   // per thread and destination: count, then running offset
  __shared__ int32_t dest_slot[kSendMaxChunk];
  __shared__ int8_t dest_rank[kSendMaxChunk];
  __shared__ int32_t cta_base[kSendMaxRanks], recv_base[kSendMaxRanks], total[kSendMaxRanks];
  const int tid = threadIdx.x, G = p.G, C = gridDim.x;
  const int R = p.T * p.K;
  const int chunk = (R + C - 1) / C;
  const int r0 = blockIdx.x * chunk;
  const int n = max(0, min(R, r0 + chunk) - r0);
  const int per = (chunk + kSendThreads - 1) / kSendThreads;   // consecutive pairs owned by one thread
  const int epoch = *p.epoch;
  const int n_exp = p.e_local * G;

  // 1. destination of every pair of this CTA's chunk; counts per (thread, destination)
  for (int d = 0; d < G; ++d) tcnt[tid][d] = 0;
  for (int j = 0; j < per; ++j) {
    const int i = tid * per + j;
    if (i < n) {
      const int e = p.topk_ids[r0 + i];
      const int d = (e >= 0 && e < n_exp) ? e / p.e_local : -1;
      dest_rank[i] = static_cast<int8_t>(d);
      if (d >= 0) tcnt[tid][d]++;
    }
  }
  __syncthreads();
  if (tid < G) {
    int run = 0;
    for (int t = 0; t < kSendThreads; ++t) {
      const int v = tcnt[t][tid];
      tcnt[t][tid] = run;
      run += v;
    }
    p.cta_counts[blockIdx.x * G + tid] = run;
  }
  // 2. all CTAs of this kernel meet (they are co-resident: at most one per SM, small footprint)
  __syncthreads();
  if (tid == 0) {
    __threadfence();
    atomicAdd(&p.sync[0], 1);
    const long long t0 = clock64();
    while (atomicAdd(&p.sync[0], 0) < C) {
      if (clock64() - t0 > p.limit) {
        atomicExch(p.status, 0x310);
        break;
      }
      __nanosleep(32);
    }
    __threadfence();
  }
  __syncthreads();
  // 3. offsets of this CTA inside each destination's group; totals; CTA 0 publishes the totals
  if (tid < G) {
    int before = 0, all = 0;
    for (int c = 0; c < C; ++c) {
      const int v = __ldcg(&p.cta_counts[c * G + tid]);
      if (c < static_cast<int>(blockIdx.x)) before += v;
      all += v;
    }
    cta_base[tid] = before;
    total[tid] = all;
  }
  __syncthreads();
  if (blockIdx.x == 0) {
    for (int i = tid; i < G * G; i += kSendThreads) {
      const int peer = i / G, d = i % G;
      peer_ptr<int32_t>(p.peer_base, peer, p.lay.matrix)[p.me * G + d] = total[d];
    }
    __syncthreads();          // the release store below orders the CTA's count stores before the flag
    if (tid < G) st_release_sys(peer_ptr<int32_t>(p.peer_base, tid, p.lay.flags) + p.me, epoch);
  }
  // 4. everybody's counts
  wait_flags(peer_ptr<int32_t>(p.peer_base, p.me, p.lay.flags), p.sync + 2, G, epoch, p.limit, p.status);
  const int32_t* matrix = peer_ptr<int32_t>(p.peer_base, p.me, p.lay.matrix);
  if (tid < G) {
    int base = 0;
    for (int s2 = 0; s2 < p.me; ++s2) base += __ldcg(&matrix[s2 * G + tid]);
    recv_base[tid] = base;
  }
  if (blockIdx.x == 0 && tid == 0) {
    int nr = 0;
    for (int s2 = 0; s2 < G; ++s2) nr += __ldcg(&matrix[s2 * G + p.me]);
    *p.n_recv_dev = nr;
  }
  __syncthreads();
  // 5. receive slot of every pair (stable: CTA, thread, position)
  for (int j = 0; j < per; ++j) {
    const int i = tid * per + j;
    if (i < n) {
      const int d = dest_rank[i];
      dest_slot[i] = d >= 0 ? recv_base[d] + cta_base[d] + tcnt[tid][d]++ : -1;
    }
  }
  __syncthreads();
  // 6. rows and their metadata into the owners' receive arrays (plain peer stores)
  const int nvec = p.row_vecs;
  for (int idx = tid; idx < n * nvec; idx += kSendThreads) {
    const int i = idx / nvec, v = idx - i * nvec;
    const int d = dest_rank[i], dst = dest_slot[i];
    if (d < 0 || dst >= p.lay.recv_cap) continue;
    const int r = r0 + i;
    peer_ptr<uint4>(p.peer_base, d, p.lay.rows)[static_cast<size_t>(dst) * nvec + v] =
        p.x[static_cast<size_t>(r / p.K) * nvec + v];
  }
  for (int i = tid; i < n; i += kSendThreads) {
    const int d = dest_rank[i], dst = dest_slot[i];
    if (d < 0 || dst >= p.lay.recv_cap) continue;
    const int r = r0 + i;
    for (int w = 0; w < p.scale_words; ++w)
      peer_ptr<uint32_t>(p.peer_base, d, p.lay.row_scales)[static_cast<size_t>(dst) * p.scale_words + w] =
          p.x_scale[static_cast<size_t>(r / p.K) * p.scale_words + w];
    peer_ptr<int32_t>(p.peer_base, d, p.lay.ids)[dst] = p.topk_ids[r] % p.e_local;
    peer_ptr<float>(p.peer_base, d, p.lay.weights)[dst] = p.topk_w[r];
    peer_ptr<int2>(p.peer_base, d, p.lay.src)[dst] = make_int2(p.me, r);
  }
  // 7. the last CTA to finish tells every rank that this rank's rows are complete (one
  //    system-scope fence for the whole grid: the last CTA's, after it has seen every count)
  __syncthreads();
  if (tid == 0) {
    __threadfence();
    const int prev = atomicAdd(&p.sync[1], 1);
    if (prev == C - 1) {
      p.sync[0] = 0;
      p.sync[1] = 0;
      fence_acq_rel_sys();
      for (int peer = 0; peer < G; ++peer)
        st_relaxed_sys(peer_ptr<int32_t>(p.peer_base, peer, p.lay.flags_dispatch) + p.me, epoch);
    }
  }
}

// The same step with one row per (token, owner rank): a token whose K experts live on fewer than K
// ranks crosses the wire once per rank, with its K-wide list of local expert ids (-1 where the
// expert lives elsewhere), weights and return slots, and the owner's operator multiplies it for
// every listed expert.  One token per thread (at most kSendThreads tokens per CTA).
__global__ void __launch_bounds__(kSendThreads)
ep_send_dedup_kernel(const EpSendParams p) {
  __shared__ int32_t tcnt[kSendThreads][kSendMaxRanks];      // per token and destination: 0/1, then running offset
  __shared__ int32_t slot_of[kSendThreads][kSendMaxRanks];   // receive slot of (token, destination), -1 = not sent there
  __shared__ int32_t cta_base[kSendMaxRanks], recv_base[kSendMaxRanks], total[kSendMaxRanks];
  const int tid = threadIdx.x, G = p.G, C = gridDim.x;
  const int chunk = (p.T + C - 1) / C;             // <= kSendThreads (checked by the host)
  const int t0 = blockIdx.x * chunk;
  const int n = max(0, min(p.T, t0 + chunk) - t0);
  const int epoch = *p.epoch;
  const int n_exp = p.e_local * G;

  // 1. owner ranks of this thread's token
  uint32_t mask = 0;
  if (tid < n) {
    for (int k = 0; k < p.K; ++k) {
      const int e = p.topk_ids[(t0 + tid) * p.K + k];
      if (e >= 0 && e < n_exp) mask |= 1u << (e / p.e_local);
    }
  }
  for (int d = 0; d < G; ++d) tcnt[tid][d] = static_cast<int32_t>((mask >> d) & 1u);
  __syncthreads();
  if (tid < G) {
    int run = 0;
    for (int t = 0; t < kSendThreads; ++t) {
      const int v = tcnt[t][tid];
      tcnt[t][tid] = run;
      run += v;
    }
    p.cta_counts[blockIdx.x * G + tid] = run;
  }
  // 2. all CTAs of this kernel meet (they are co-resident: at most one per SM)
  __syncthreads();
  if (tid == 0) {
    __threadfence();
    atomicAdd(&p.sync[0], 1);
    const long long t_start = clock64();
    while (atomicAdd(&p.sync[0], 0) < C) {
      if (clock64() - t_start > p.limit) {
        atomicExch(p.status, 0x310);
        break;
      }
      __nanosleep(32);
    }
    __threadfence();
  }
  __syncthreads();
  // 3. offsets of this CTA inside each destination's group; totals; CTA 0 publishes the totals
  if (tid < G) {
    int before = 0, all = 0;
    for (int c = 0; c < C; ++c) {
      const int v = __ldcg(&p.cta_counts[c * G + tid]);
      if (c < static_cast<int>(blockIdx.x)) before += v;
      all += v;
    }
    cta_base[tid] = before;
    total[tid] = all;
  }
  __syncthreads();
  if (blockIdx.x == 0) {
    for (int i = tid; i < G * G; i += kSendThreads) {
      const int peer = i / G, d = i % G;
      peer_ptr<int32_t>(p.peer_base, peer, p.lay.matrix)[p.me * G + d] = total[d];
    }
    __syncthreads();
    if (tid < G) st_release_sys(peer_ptr<int32_t>(p.peer_base, tid, p.lay.flags) + p.me, epoch);
  }
  // 4. everybody's counts
  wait_flags(peer_ptr<int32_t>(p.peer_base, p.me, p.lay.flags), p.sync + 2, G, epoch, p.limit, p.status);
  const int32_t* matrix = peer_ptr<int32_t>(p.peer_base, p.me, p.lay.matrix);
  if (tid < G) {
    int base = 0;
    for (int s2 = 0; s2 < p.me; ++s2) base += __ldcg(&matrix[s2 * G + tid]);
    recv_base[tid] = base;
  }
  if (blockIdx.x == 0 && tid == 0) {
    int nr = 0;
    for (int s2 = 0; s2 < G; ++s2) nr += __ldcg(&matrix[s2 * G + p.me]);
    *p.n_recv_dev = nr;
  }
  __syncthreads();
  // 5. receive slot of every (token, destination)
  for (int d = 0; d < G; ++d)
    slot_of[tid][d] = ((mask >> d) & 1u) ? recv_base[d] + cta_base[d] + tcnt[tid][d] : -1;
  __syncthreads();
  // 6. one warp per (token, destination): the row, its scales, the K-wide metadata
  const int warp = tid >> 5, lane = tid & 31;
  for (int pd = warp; pd < n * G; pd += kSendThreads / 32) {
    const int i = pd / G, d = pd - i * G;
    const int dst = slot_of[i][d];
    if (dst < 0 || dst >= p.lay.recv_cap) continue;
    const int t = t0 + i;
    uint4* rows = peer_ptr<uint4>(p.peer_base, d, p.lay.rows) + static_cast<size_t>(dst) * p.row_vecs;
    const uint4* src_row = p.x + static_cast<size_t>(t) * p.row_vecs;
    for (int v = lane; v < p.row_vecs; v += 32) rows[v] = src_row[v];
    for (int w = lane; w < p.scale_words; w += 32)
      peer_ptr<uint32_t>(p.peer_base, d, p.lay.row_scales)[static_cast<size_t>(dst) * p.scale_words + w] =
          p.x_scale[static_cast<size_t>(t) * p.scale_words + w];
    for (int k = lane; k < p.K; k += 32) {
      const int r = t * p.K + k;
      const int e = p.topk_ids[r];
      const bool here = e >= 0 && e < n_exp && e / p.e_local == d;
      const size_t o = static_cast<size_t>(dst) * p.K + k;
      peer_ptr<int32_t>(p.peer_base, d, p.lay.ids)[o] = here ? e % p.e_local : -1;
      peer_ptr<float>(p.peer_base, d, p.lay.weights)[o] = p.topk_w[r];
      peer_ptr<int32_t>(p.peer_base, d, p.lay.src)[o] = here ? r : -1;
    }
    if (lane == 0) peer_ptr<int32_t>(p.peer_base, d, p.lay.src_rank)[dst] = p.me;
  }
  // 7. the last CTA to finish tells every rank that this rank's rows are complete
  __syncthreads();
  if (tid == 0) {
    __threadfence();
    const int prev = atomicAdd(&p.sync[1], 1);
    if (prev == C - 1) {
      p.sync[0] = 0;
      p.sync[1] = 0;
      fence_acq_rel_sys();
      for (int peer = 0; peer < G; ++peer)
        st_relaxed_sys(peer_ptr<int32_t>(p.peer_base, peer, p.lay.flags_dispatch) + p.me, epoch);
    }
  }
}

// Return addresses of the de-duplicated step: entry (row, k) of the received rows.
__global__ void __launch_bounds__(256)
ep_recv_ready_dedup_kernel(int H, int K, const int32_t* __restrict__ n_recv_dev,
                           const uint64_t* __restrict__ peer_base, fmoe_ep_layout_c lay, int me, int G,
                           const int32_t* __restrict__ epoch, uint64_t* __restrict__ row_ptrs,
                           int32_t* __restrict__ scratch, int32_t* __restrict__ status, long long limit) {
  wait_flags(peer_ptr<int32_t>(peer_base, me, lay.flags_dispatch), scratch + 3, G, *epoch, limit, status);
  const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  const long long row = i / K;
  if (row >= *n_recv_dev || row >= lay.recv_cap) return;
  const int s = __ldcg(peer_ptr<int32_t>(peer_base, me, lay.src) + i);
  if (s < 0) return;                       // this expert of the token lives on another rank: never read
  const int from = __ldcg(peer_ptr<int32_t>(peer_base, me, lay.src_rank) + row);
  // never follow a bad return address: such a row goes to a scratch row of this rank instead
  const bool ok = from >= 0 && from < G && s < lay.send_cap;
  row_ptrs[i] = ok ? peer_base[from] + lay.back + static_cast<uint64_t>(s) * H * 2 : peer_base[me] + lay.rows;
  if (!ok) atomicExch(status, 0x320);
}

__global__ void __launch_bounds__(256)
ep_recv_ready_kernel(int H, const int32_t* __restrict__ n_recv_dev, const uint64_t* __restrict__ peer_base,
                     fmoe_ep_layout_c lay, int me, int G, const int32_t* __restrict__ epoch,
                     uint64_t* __restrict__ row_ptrs, int32_t* __restrict__ scratch, int32_t* __restrict__ status,
                     long long limit) {
  wait_flags(peer_ptr<int32_t>(peer_base, me, lay.flags_dispatch), scratch + 3, G, *epoch, limit, status);
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= *n_recv_dev || i >= lay.recv_cap) return;
  const int2 s = __ldcg(peer_ptr<int2>(peer_base, me, lay.src) + i);
  // never follow a bad return address: such a row goes to a scratch row of this rank instead
  const bool ok = s.x >= 0 && s.x < G && s.y >= 0 && s.y < lay.send_cap;
  row_ptrs[i] = ok ? peer_base[s.x] + lay.back + static_cast<uint64_t>(s.y) * H * 2
                   : peer_base[me] + lay.rows;
  if (!ok) atomicExch(status, 0x320);
}

__global__ void __launch_bounds__(128)
ep_wait_combine_kernel(const int32_t* __restrict__ topk_ids, int K, int H, int E,
                       const uint64_t* __restrict__ peer_base, fmoe_ep_layout_c lay, int me, int G,
                       int32_t* __restrict__ epoch, int32_t* __restrict__ scratch, uint4* __restrict__ out,
                       int32_t* __restrict__ status, long long limit) {
  int32_t* sync_counter = scratch + 5;
  wait_flags(peer_ptr<int32_t>(peer_base, me, lay.flags_return), scratch + 4, G, *epoch, limit, status);
  const int t = blockIdx.x;
  const int nvec = H >> 3;
  const uint4* back = peer_ptr<uint4>(peer_base, me, lay.back);
  for (int i = threadIdx.x; i < nvec; i += blockDim.x) {
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int k = 0; k < K; ++k) {
      const int e = topk_ids[t * K + k];
      if (e < 0 || e >= E) continue;
      const uint4 v = __ldcg(back + (static_cast<size_t>(t) * K + k) * nvec + i);   // written by a peer: skip L1
      const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        acc[2 * j] += __uint_as_float(w[j] << 16);
        acc[2 * j + 1] += __uint_as_float(w[j] & 0xffff0000u);
      }
    }
    uint32_t o[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      __nv_bfloat162 h = __floats2bfloat162_rn(acc[2 * j], acc[2 * j + 1]);
      o[j] = *reinterpret_cast<uint32_t*>(&h);
    }
    out[static_cast<size_t>(t) * nvec + i] = make_uint4(o[0], o[1], o[2], o[3]);
  }
  // the last CTA to finish opens the next step
  __syncthreads();
  if (threadIdx.x == 0) {
    const int prev = atomicAdd(sync_counter, 1);
    if (prev == static_cast<int>(gridDim.x) - 1) {
      *sync_counter = 0;
      *epoch = *epoch + 1;
    }
  }
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

static long long wait_limit_cycles(int32_t timeout_ms) {
  // clock64 ticks at the SM clock (<= ~2 GHz): 2e6 cycles per millisecond is an upper bound
  return timeout_ms > 0 ? 2000000LL * timeout_ms : 8000000000LL;
}

static int ep_send_grid(int32_t T, int32_t K) {
  const long long R = static_cast<long long>(T) * K;
  long long c = (R + fmoe::kSendPairsPerCta - 1) / fmoe::kSendPairsPerCta;
  const int sms = fmoe::device_sm_count();
  if (c > sms) c = sms;
  return c < 1 ? 1 : static_cast<int>(c);
}

int64_t fmoe_ep_send_scratch_words(int32_t T, int32_t K, int32_t G) {
  (void)T; (void)K;
  return 8 + 256LL * (G > 0 ? G : 1);      // counters and wait words + per-CTA counts for up to 256 CTAs
}

int fmoe_ep_send(const void* x, const int32_t* topk_ids, const float* topk_weight, int32_t T, int32_t K, int32_t H,
                 int32_t experts_per_rank, const uint64_t* peer_base, const fmoe_ep_layout_c* lay, int32_t me,
                 int32_t G, int32_t* scratch, const int32_t* epoch_dev, int32_t* n_recv_dev, int32_t* status,
                 int32_t timeout_ms, void* stream) {
  if (H <= 0 || H % 8) return fmoe::fail(FMOE_ERR_UNSUPPORTED, "fmoe_ep_send: H must be a positive multiple of 8");
  return fmoe_ep_send_rows(x, 2 * H, nullptr, 0, topk_ids, topk_weight, T, K, experts_per_rank, peer_base, lay, me, G,
                           scratch, epoch_dev, n_recv_dev, status, timeout_ms, stream);
}

int fmoe_ep_send_rows(const void* x, int32_t row_bytes, const void* row_scales, int32_t scale_row_bytes,
                      const int32_t* topk_ids, const float* topk_weight, int32_t T, int32_t K,
                      int32_t experts_per_rank, const uint64_t* peer_base, const fmoe_ep_layout_c* lay, int32_t me,
                      int32_t G, int32_t* scratch, const int32_t* epoch_dev, int32_t* n_recv_dev, int32_t* status,
                      int32_t timeout_ms, void* stream) {
  if (!x || !topk_ids || !topk_weight || !peer_base || !lay || !scratch || !epoch_dev || !n_recv_dev || !status)
    return fmoe::fail(FMOE_ERR_INVALID_ARG, "fmoe_ep_send: a required pointer is null");
  if (G <= 0 || G > fmoe::kSendMaxRanks || me < 0 || me >= G)
    return fmoe::fail(FMOE_ERR_INVALID_ARG, "fmoe_ep_send: rank %d / world %d out of range (at most %d ranks)", me, G,
                      fmoe::kSendMaxRanks);
  if (row_bytes <= 0 || row_bytes % 16 || T <= 0 || K <= 0 || experts_per_rank <= 0 || timeout_ms < 0)
    return fmoe::fail(FMOE_ERR_UNSUPPORTED, "fmoe_ep_send: row bytes must be a positive multiple of 16; T, K, experts_per_rank positive");
  if (scale_row_bytes < 0 || scale_row_bytes % 4 || (scale_row_bytes > 0 && !row_scales))
    return fmoe::fail(FMOE_ERR_INVALID_ARG, "fmoe_ep_send: scale row bytes must be a multiple of 4 and come with row_scales");
  const int grid = ep_send_grid(T, K);
  if ((static_cast<long long>(T) * K + grid - 1) / grid > fmoe::kSendMaxChunk)
    return fmoe::fail(FMOE_ERR_UNSUPPORTED, "fmoe_ep_send: at most %d routed pairs per rank", grid * fmoe::kSendMaxChunk);
  fmoe::EpSendParams p;
  p.x = reinterpret_cast<const uint4*>(x);
  p.x_scale = reinterpret_cast<const uint32_t*>(row_scales);
  p.row_vecs = row_bytes / 16; p.scale_words = scale_row_bytes / 4;
  p.topk_ids = topk_ids; p.topk_w = topk_weight;
  p.T = T; p.K = K; p.e_local = experts_per_rank;
  p.peer_base = peer_base; p.lay = *lay; p.me = me; p.G = G;
  p.sync = scratch; p.cta_counts = scratch + 8;
  p.epoch = epoch_dev; p.n_recv_dev = n_recv_dev; p.status = status;
  p.limit = wait_limit_cycles(timeout_ms);
  fmoe::ep_send_kernel<<<grid, fmoe::kSendThreads, 0, static_cast<cudaStream_t>(stream)>>>(p);
  return fmoe::launch_status("fmoe_ep_send");
}

int fmoe_ep_send_rows_dedup(const void* x, int32_t row_bytes, const void* row_scales, int32_t scale_row_bytes,
                            const int32_t* topk_ids, const float* topk_weight, int32_t T, int32_t K,
                            int32_t experts_per_rank, const uint64_t* peer_base, const fmoe_ep_layout_c* lay,
                            int32_t me, int32_t G, int32_t* scratch, const int32_t* epoch_dev, int32_t* n_recv_dev,
                            int32_t* status, int32_t timeout_ms, void* stream) {
  if (!x || !topk_ids || !topk_weight || !peer_base || !lay || !scratch || !epoch_dev || !n_recv_dev || !status)
    return fmoe::fail(FMOE_ERR_INVALID_ARG, "fmoe_ep_send_rows_dedup: a required pointer is null");
  if (G <= 0 || G > fmoe::kSendMaxRanks || me < 0 || me >= G)
    return fmoe::fail(FMOE_ERR_INVALID_ARG, "fmoe_ep_send_rows_dedup: rank %d / world %d out of range (at most %d ranks)",
                      me, G, fmoe::kSendMaxRanks);
  if (row_bytes <= 0 || row_bytes % 16 || T <= 0 || K <= 0 || experts_per_rank <= 0 || timeout_ms < 0)
    return fmoe::fail(FMOE_ERR_UNSUPPORTED, "fmoe_ep_send_rows_dedup: row bytes must be a positive multiple of 16; T, K, experts_per_rank positive");
  if (scale_row_bytes < 0 || scale_row_bytes % 4 || (scale_row_bytes > 0 && !row_scales))
    return fmoe::fail(FMOE_ERR_INVALID_ARG, "fmoe_ep_send_rows_dedup: scale row bytes must be a multiple of 4 and come with row_scales");
  const int sms = fmoe::device_sm_count();
  const int grid = T < sms ? T : sms;
  if ((T + grid - 1) / grid > fmoe::kSendThreads)
    return fmoe::fail(FMOE_ERR_UNSUPPORTED, "fmoe_ep_send_rows_dedup: at most %d tokens per rank", grid * fmoe::kSendThreads);
  fmoe::EpSendParams p;
  p.x = reinterpret_cast<const uint4*>(x);
  p.x_scale = reinterpret_cast<const uint32_t*>(row_scales);
  p.row_vecs = row_bytes / 16; p.scale_words = scale_row_bytes / 4;
  p.topk_ids = topk_ids; p.topk_w = topk_weight;
  p.T = T; p.K = K; p.e_local = experts_per_rank;
  p.peer_base = peer_base; p.lay = *lay; p.me = me; p.G = G;
  p.sync = scratch; p.cta_counts = scratch + 8;
  p.epoch = epoch_dev; p.n_recv_dev = n_recv_dev; p.status = status;
  p.limit = wait_limit_cycles(timeout_ms);
  fmoe::ep_send_dedup_kernel<<<grid, fmoe::kSendThreads, 0, static_cast<cudaStream_t>(stream)>>>(p);
  return fmoe::launch_status("fmoe_ep_send_rows_dedup");
}

int fmoe_ep_recv_ready_dedup(int32_t H, int32_t K, const int32_t* n_recv_dev, const uint64_t* peer_base,
                             const fmoe_ep_layout_c* lay, int32_t me, int32_t G, const int32_t* epoch_dev,
                             uint64_t* row_ptrs, int32_t* scratch, int32_t* status, int32_t timeout_ms, void* stream) {
  if (!n_recv_dev || !peer_base || !lay || !epoch_dev || !row_ptrs || !scratch || !status)
    return fmoe::fail(FMOE_ERR_INVALID_ARG, "fmoe_ep_recv_ready_dedup: a required pointer is null");
  if (G <= 0 || G > fmoe::kSendMaxRanks || me < 0 || me >= G || H <= 0 || K <= 0 || timeout_ms < 0)
    return fmoe::fail(FMOE_ERR_INVALID_ARG, "fmoe_ep_recv_ready_dedup: bad arguments (rank %d, world %d, H %d, K %d)", me,
                      G, H, K);
  if (lay->recv_cap <= 0) return FMOE_OK;
  const unsigned grid = static_cast<unsigned>((lay->recv_cap * K + 255) / 256);
  fmoe::ep_recv_ready_dedup_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      H, K, n_recv_dev, peer_base, *lay, me, G, epoch_dev, row_ptrs, scratch, status, wait_limit_cycles(timeout_ms));
  return fmoe::launch_status("fmoe_ep_recv_ready_dedup");
}

int fmoe_ep_recv_ready(int32_t H, const int32_t* n_recv_dev, const uint64_t* peer_base, const fmoe_ep_layout_c* lay,
                       int32_t me, int32_t G, const int32_t* epoch_dev, uint64_t* row_ptrs, int32_t* scratch,
                       int32_t* status, int32_t timeout_ms, void* stream) {
  if (!n_recv_dev || !peer_base || !lay || !epoch_dev || !row_ptrs || !scratch || !status)
    return fmoe::fail(FMOE_ERR_INVALID_ARG, "fmoe_ep_recv_ready: a required pointer is null");
  if (G <= 0 || G > fmoe::kSendMaxRanks || me < 0 || me >= G || H <= 0 || timeout_ms < 0)
    return fmoe::fail(FMOE_ERR_INVALID_ARG, "fmoe_ep_recv_ready: bad arguments (rank %d, world %d, H %d)", me, G, H);
  if (lay->recv_cap <= 0) return FMOE_OK;
  const unsigned grid = static_cast<unsigned>((lay->recv_cap + 255) / 256);
  fmoe::ep_recv_ready_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      H, n_recv_dev, peer_base, *lay, me, G, epoch_dev, row_ptrs, scratch, status, wait_limit_cycles(timeout_ms));
  return fmoe::launch_status("fmoe_ep_recv_ready");
}

int fmoe_ep_wait_combine(const int32_t* topk_ids, int32_t T, int32_t K, int32_t H, int32_t num_experts,
                         const uint64_t* peer_base, const fmoe_ep_layout_c* lay, int32_t me, int32_t G,
                         int32_t* epoch_dev, int32_t* scratch, void* out, int32_t* status, int32_t timeout_ms,
                         void* stream) {
  if (!topk_ids || !peer_base || !lay || !epoch_dev || !scratch || !out || !status)
    return fmoe::fail(FMOE_ERR_INVALID_ARG, "fmoe_ep_wait_combine: a required pointer is null");
  if (G <= 0 || G > fmoe::kSendMaxRanks || me < 0 || me >= G || T <= 0 || K <= 0 || H <= 0 || H % 8 || timeout_ms < 0)
    return fmoe::fail(FMOE_ERR_INVALID_ARG, "fmoe_ep_wait_combine: bad arguments (rank %d, world %d, T %d, K %d, H %d)", me,
                      G, T, K, H);
  fmoe::ep_wait_combine_kernel<<<T, 128, 0, static_cast<cudaStream_t>(stream)>>>(
      topk_ids, K, H, num_experts, peer_base, *lay, me, G, epoch_dev, scratch, reinterpret_cast<uint4*>(out),
      status, wait_limit_cycles(timeout_ms));
  return fmoe::launch_status("fmoe_ep_wait_combine");
}

}  // extern "C"
