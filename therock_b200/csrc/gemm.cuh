// Expert-grouped GEMMs for the fused-MoE operator on sm_100a: the single-CTA kernel described
// here and a CTA-pair variant (cta_group::2) further down; the block-scaled fp8 kernels are in
// gemm_block.cuh.
//
// One persistent CTA per SM walks a list of (expert, n-block, m-block) tiles.  Every tile
// is D[128 x 256] = A[128 x K] * B[256 x K]^T with
//   A  = 128 consecutive sorted rows (one moe_sorting block, all of one expert),
//   B  = two 128-row slabs of that expert's weight matrix (gate rows + up rows for the
//        first GEMM, two consecutive row slabs for the second).
// Operands arrive through TMA into a 4-stage shared-memory ring (128-byte swizzle),
// tcgen05.mma accumulates in tensor memory (two 256-column accumulators so the epilogue of
// tile i overlaps the main loop of tile i+1), and four epilogue warps read the accumulator
// back with tcgen05.ld and apply the fused epilogue.
//
// Warp roles (192 threads): warp 0 = TMA producer, warp 1 = MMA issuer + TMEM owner,
// warps 2..5 = epilogue (warp w may touch TMEM lanes 32*(w%4) .. +31).
#pragma once

#include <cuda_bf16.h>

#include "ptx.cuh"

namespace fmoe {

constexpr int kBlockM = 128;        // rows per tile == moe_sorting block
constexpr int kTileN = 256;         // accumulator columns per tile
constexpr int kSlabRows = 128;      // rows per B slab (two slabs per tile)
constexpr int kStageKBytes = 128;   // bytes of K per pipeline stage (one swizzle row)
constexpr int kStages = 4;
constexpr int kABytes = kBlockM * kStageKBytes;            // 16 KiB
constexpr int kBBytes = kTileN * kStageKBytes;             // 32 KiB
constexpr int kStageBytes = kABytes + kBBytes;             // 48 KiB
constexpr int kGemmThreads = 192;
constexpr int kTmemCols = 512;
constexpr int kSmemMisc = 8192;          // barriers + per-expert block table (<= 1025 ints)
constexpr int kEpiStageReserve = 4 * 32 * 36 * 4;   // per-warp staging of the epilogue (see epilogue_tile)
constexpr int kGemmSmemBytes = kStages * kStageBytes + kSmemMisc + kEpiStageReserve + 1024;  // +1024 alignment slack

enum : int { kEpiSiluMul = 1, kEpiScaledSlots = 2, kEpiSilu = 3 };

// Device status codes written to the workspace status word.
enum : int { kStatusOk = 0, kStatusGemmTimeout = 0x100 };

struct GemmParams {
  const int* mblk_cum;          // [E+1] cumulative 128-row blocks per expert (from moe_sorting)
  int num_experts;
  int n_blocks;                 // tiles along N per expert
  int k_iters;                  // ceil(K_bytes / 128)
  int b_rows_per_expert;        // rows of the B matrix per expert
  int n_stride;                 // first-slab row step per n-block
  int second_slab_offset;       // row distance from the first slab to the second
  const int* sorted_rows;       // [cap] flat (token*K + k) per sorted slot, -1 = pad
  const float* sorted_weights;  // [cap]
  const float* a_scale;         // [cap] per-sorted-row activation scale, or nullptr
  const float* b_scale;         // [E * b_rows_per_expert] per-output-channel scale, or nullptr
  void* out;                    // kEpiSiluMul: bf16 [cap, ld_out]; kEpiScaledSlots: f32 or bf16 [T*K, ld_out]
  int ld_out;                   // elements per output row
  int out_bf16;                 // kEpiScaledSlots: 1 = weighted rows are rounded to bf16
  int64_t out_rows;             // rows of `out` (bound for the checked build)
  const uint64_t* row_ptrs;     // kEpiScaledSlots with bf16 rows: destination address of each routed pair's row
                                // (may be peer memory) instead of out + pair * ld_out; nullptr = contiguous
  const uint64_t* done_addrs;   // completion signal: the last CTA to finish writes *done_value to these
  const int* done_value;        // addresses (release, system scope); nullptr = none
  int* done_counter;
  int done_count;
  int* status;                  // device status word
  uint64_t desc_template;       // shared-memory matrix descriptor without the address
  uint32_t idesc;               // tcgen05 instruction descriptor
  int b_tiled_kb;               // 0: B is row-major; > 0: B is stored as contiguous 128 x 128-byte
                                // tiles and this is the number of 128-byte K blocks per row
#ifdef FMOE_TIMING_SWITCHES
  uint32_t debug_flags;         // timing experiments only (results are invalid when set): bit 0 = the
                                // epilogue skips its work (block-scaled kernel: no promotion
                                // FMAs), bit 1 = no MMA is issued; block-scaled kernel only:
                                // bit 2 = no TMEM loads, bit 4 = no final stores,
                                // bit 5 = no TMA loads (the MMAs run on whatever shared memory holds)
#endif
};

// The timing switches exist only in a library built with -DFMOE_TIMING_SWITCHES; in the
// product build the tests below are constant false and the compiler drops them.
#ifdef FMOE_TIMING_SWITCHES
#define FMOE_DBG(p, bits) (((p).debug_flags & (bits)) != 0)
#else
#define FMOE_DBG(p, bits) false
#endif

// Checked build (-DFMOE_BOUNDS_CHECKS): every computed output row is compared with its bound
// before the store; a violation stores a code in the status word instead of writing.
enum : int { kStatusBoundsGemm = 0x400 };
#ifdef FMOE_BOUNDS_CHECKS
#define FMOE_ROW_OK(p, r) ((r) < (p).out_rows ? true : (atomicExch((p).status, kStatusBoundsGemm), false))
#else
#define FMOE_ROW_OK(p, r) true
#endif

struct TileCoord {
  int expert, m_blk, n_blk;
};

// tile -> (expert, n-block, m-block): experts in order, then n-blocks, then that expert's
// m-blocks fastest, so CTAs running side by side share the same weight slabs through L2.
__device__ __forceinline__ TileCoord decode_tile(int tile, const int* cum, int E,
                                                 int n_blocks) {
  int lo = 1, hi = E;
  while (lo < hi) {
    int mid = (lo + hi) >> 1;
    if (cum[mid] * n_blocks > tile) hi = mid; else lo = mid + 1;
  }
  TileCoord t;
  t.expert = lo - 1;
  int base = cum[t.expert];
  int cnt = cum[t.expert + 1] - base;
  int local = tile - base * n_blocks;
  t.n_blk = local / cnt;
  t.m_blk = base + local % cnt;
  return t;
}

// Completion signal of a whole grid: every CTA calls this after its last store (all threads,
// after a CTA-wide barrier).  The last CTA to arrive publishes *done_value to the given
// addresses, which may lie in other GPUs' memory, so their kernels can wait for this grid's
// rows without a further launch.
__device__ __forceinline__ void grid_done_signal(const GemmParams& p) {
  if (p.done_addrs == nullptr || threadIdx.x != 0) return;
  // This CTA's stores (seen through the barrier) are ordered before its count at device scope;
  // the one system-scope fence of the grid is the last CTA's, which has observed every count.
  __threadfence();
  const int prev = atomicAdd(p.done_counter, 1);
  if (prev != static_cast<int>(gridDim.x) - 1) return;
  ptx::fence_acq_rel_sys();
  const int v = *p.done_value;
  for (int i = 0; i < p.done_count; ++i)
    asm volatile("st.relaxed.sys.global.s32 [%0], %1;" ::"l"(p.done_addrs[i]), "r"(v) : "memory");
  *p.done_counter = 0;                            // ready for the next launch
}

// SiLU with the fast exponential and division (a few ulp; far inside the bf16 rounding of y).
// TMA coordinates of the 128-row B slab starting at row `b_row` for K stage `k`.
__device__ __forceinline__ void b_coords(const GemmParams& p, int b_row, int k, int elems_per_stage, int& x, int& y) {
  if (p.b_tiled_kb > 0) {
    x = 0;
    y = ((b_row >> 7) * p.b_tiled_kb + k) << 7;      // tile index * 128 rows of 128 bytes
  } else {
    x = k * elems_per_stage;
    y = b_row;
  }
}

__device__ __forceinline__ float silu(float g) { return __fdividef(g, 1.0f + __expf(-g)); }

// Per-warp staging area for the epilogue's transposed stores: 32 rows x 36 words.
constexpr int kStageWordsPerRow = 36;
constexpr int kEpiStageBytesPerWarp = 32 * kStageWordsPerRow * 4;     // 4608
constexpr int kEpiStageBytes = 4 * kEpiStageBytesPerWarp;             // four epilogue warps

// Fused epilogue of one 128 x 256 accumulator held in TMEM (this thread owns one row).
//   kEpiSiluMul    : columns 0..127 gate, 128..255 up -> bf16 y[slot, n_blk*128 ..] = SiLU(g)*u
//   kEpiScaledSlots: 256 output channels -> f32 slots[row, n_blk*256 ..] = w * acc
//   kEpiSilu       : gate-only first GEMM, 256 channels -> bf16 y[slot, n_blk*256 ..] = SiLU(acc)
// fp8: acc is first multiplied by the row's activation scale and the channel's weight scale.
// A thread computes 32 consecutive columns of its own row per step.  Storing them directly
// would make every warp store touch 32 rows with 16 bytes each; instead the warp transposes
// the 32 x 32 block through its private shared-memory area (`stage`, conflict-free 16-byte
// accesses) and writes whole row segments: 128-byte (f32) or 64-byte (bf16) contiguous runs.
template <int kEpi>
__device__ __forceinline__ void epilogue_tile(const GemmParams& p, uint32_t t_row, int slot, int n_blk,
                                              const float* bs0, const float* bs1, float a_s,
                                              uint32_t* stage) {
  const int lane = threadIdx.x & 31;
  const int row = p.sorted_rows[slot];               // flat (token, k) index, < 0 for a pad slot
  // a warp whose 32 rows are all padding has nothing to store: it skips the tensor-memory reads too
  if (__ballot_sync(0xffffffffu, row >= 0) == 0u) return;
  if (kEpi == kEpiSiluMul) {
    // pad slots carry no token: their rows of y are never used, so they are not stored
    __nv_bfloat16* ybase = reinterpret_cast<__nv_bfloat16*>(p.out) + n_blk * kSlabRows;
    const int slot0 = slot - lane;                   // first sorted slot of this warp
    uint32_t g[2][32], u[2][32];
    ptx::tmem_ld_32x32(t_row, g[0]);
    ptx::tmem_ld_32x32(t_row + kSlabRows, u[0]);
#pragma unroll
    for (int c = 0; c < kSlabRows / 32; ++c) {
      const int cur = c & 1;
      ptx::tmem_ld_wait();
      if (c + 1 < kSlabRows / 32) {
        ptx::tmem_ld_32x32(t_row + (c + 1) * 32, g[cur ^ 1]);
        ptx::tmem_ld_32x32(t_row + kSlabRows + (c + 1) * 32, u[cur ^ 1]);
      }
      uint32_t packed[16];
#pragma unroll
      for (int q = 0; q < 8; ++q) {
        float gv[4], uv[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          gv[j] = __uint_as_float(g[cur][4 * q + j]);
          uv[j] = __uint_as_float(u[cur][4 * q + j]);
        }
        if (p.b_scale != nullptr) {
          const float4 sg = __ldg(reinterpret_cast<const float4*>(bs0 + c * 32 + 4 * q));
          const float4 su = __ldg(reinterpret_cast<const float4*>(bs1 + c * 32 + 4 * q));
          gv[0] = (gv[0] * a_s) * sg.x; gv[1] = (gv[1] * a_s) * sg.y;
          gv[2] = (gv[2] * a_s) * sg.z; gv[3] = (gv[3] * a_s) * sg.w;
          uv[0] = (uv[0] * a_s) * su.x; uv[1] = (uv[1] * a_s) * su.y;
          uv[2] = (uv[2] * a_s) * su.z; uv[3] = (uv[3] * a_s) * su.w;
        }
        __nv_bfloat162 v0 = __floats2bfloat162_rn(silu(gv[0]) * uv[0], silu(gv[1]) * uv[1]);
        __nv_bfloat162 v1 = __floats2bfloat162_rn(silu(gv[2]) * uv[2], silu(gv[3]) * uv[3]);
        packed[2 * q] = *reinterpret_cast<uint32_t*>(&v0);
        packed[2 * q + 1] = *reinterpret_cast<uint32_t*>(&v1);
      }
      // own row -> staging (16 words of bf16 pairs, row pitch 20 words)
      __syncwarp();
      uint4* srow = reinterpret_cast<uint4*>(stage + lane * 20);
#pragma unroll
      for (int q = 0; q < 4; ++q)
        srow[q] = make_uint4(packed[4 * q], packed[4 * q + 1], packed[4 * q + 2], packed[4 * q + 3]);
      __syncwarp();
      // 4 lanes per row, 8 rows per store instruction: 64 contiguous bytes per row
#pragma unroll
      for (int it = 0; it < 4; ++it) {
        const int r = it * 8 + (lane >> 2);
        const int seg = lane & 3;
        const uint4 val = *reinterpret_cast<const uint4*>(stage + r * 20 + seg * 4);
        const int live_r = __shfl_sync(0xffffffffu, row, r);
        if (live_r >= 0 && FMOE_ROW_OK(p, slot0 + r))
          *reinterpret_cast<uint4*>(ybase + static_cast<size_t>(slot0 + r) * p.ld_out + c * 32 + seg * 8) = val;
      }
    }
  } else if (kEpi == kEpiSilu) {
    __nv_bfloat16* ybase = reinterpret_cast<__nv_bfloat16*>(p.out) + n_blk * kTileN;
    const int slot0 = slot - lane;
    uint32_t v[2][32];
    ptx::tmem_ld_32x32(t_row, v[0]);
#pragma unroll
    for (int c = 0; c < kTileN / 32; ++c) {
      const int cur = c & 1;
      ptx::tmem_ld_wait();
      if (c + 1 < kTileN / 32) ptx::tmem_ld_32x32(t_row + (c + 1) * 32, v[cur ^ 1]);
      uint32_t packed[16];
#pragma unroll
      for (int q = 0; q < 8; ++q) {
        float f[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) f[j] = __uint_as_float(v[cur][4 * q + j]);
        if (p.b_scale != nullptr) {
          const float4 sc = __ldg(reinterpret_cast<const float4*>(bs0 + c * 32 + 4 * q));
          f[0] = (f[0] * a_s) * sc.x; f[1] = (f[1] * a_s) * sc.y;
          f[2] = (f[2] * a_s) * sc.z; f[3] = (f[3] * a_s) * sc.w;
        }
        __nv_bfloat162 v0 = __floats2bfloat162_rn(silu(f[0]), silu(f[1]));
        __nv_bfloat162 v1 = __floats2bfloat162_rn(silu(f[2]), silu(f[3]));
        packed[2 * q] = *reinterpret_cast<uint32_t*>(&v0);
        packed[2 * q + 1] = *reinterpret_cast<uint32_t*>(&v1);
      }
      __syncwarp();
      uint4* srow = reinterpret_cast<uint4*>(stage + lane * 20);
#pragma unroll
      for (int q = 0; q < 4; ++q)
        srow[q] = make_uint4(packed[4 * q], packed[4 * q + 1], packed[4 * q + 2], packed[4 * q + 3]);
      __syncwarp();
#pragma unroll
      for (int it = 0; it < 4; ++it) {
        const int r = it * 8 + (lane >> 2);
        const int seg = lane & 3;
        const uint4 val = *reinterpret_cast<const uint4*>(stage + r * 20 + seg * 4);
        const int live_r = __shfl_sync(0xffffffffu, row, r);
        if (live_r >= 0 && FMOE_ROW_OK(p, slot0 + r))
          *reinterpret_cast<uint4*>(ybase + static_cast<size_t>(slot0 + r) * p.ld_out + c * 32 + seg * 8) = val;
      }
    }
  } else {
    const float w = p.sorted_weights[slot];
    float* obase = reinterpret_cast<float*>(p.out) + n_blk * kTileN;
    uint32_t v[2][32];
    ptx::tmem_ld_32x32(t_row, v[0]);
#pragma unroll
    for (int c = 0; c < kTileN / 32; ++c) {
      const int cur = c & 1;
      ptx::tmem_ld_wait();
      if (c + 1 < kTileN / 32) ptx::tmem_ld_32x32(t_row + (c + 1) * 32, v[cur ^ 1]);
      __syncwarp();
      float4* srow = reinterpret_cast<float4*>(stage + lane * kStageWordsPerRow);
#pragma unroll
      for (int q = 0; q < 8; ++q) {
        float f[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) f[j] = __uint_as_float(v[cur][4 * q + j]);
        if (p.b_scale != nullptr) {
          // second GEMM: the tile's 256 columns are 256 consecutive output channels
          const float4 sc = __ldg(reinterpret_cast<const float4*>(bs0 + c * 32 + 4 * q));
          f[0] = (f[0] * a_s) * sc.x; f[1] = (f[1] * a_s) * sc.y;
          f[2] = (f[2] * a_s) * sc.z; f[3] = (f[3] * a_s) * sc.w;
        }
        srow[q] = make_float4(w * f[0], w * f[1], w * f[2], w * f[3]);
      }
      __syncwarp();
      if (p.out_bf16) {
        // bf16 partial rows: 4 lanes per row, 8 rows per store instruction, 64 bytes per row
        __nv_bfloat16* hbase = reinterpret_cast<__nv_bfloat16*>(p.out) + n_blk * kTileN;
#pragma unroll
        for (int it = 0; it < 4; ++it) {
          const int r = it * 8 + (lane >> 2);
          const int seg = lane & 3;
          const float4 v0 = *reinterpret_cast<const float4*>(stage + r * kStageWordsPerRow + seg * 8);
          const float4 v1 = *reinterpret_cast<const float4*>(stage + r * kStageWordsPerRow + seg * 8 + 4);
          __nv_bfloat162 h0 = __floats2bfloat162_rn(v0.x, v0.y), h1 = __floats2bfloat162_rn(v0.z, v0.w);
          __nv_bfloat162 h2 = __floats2bfloat162_rn(v1.x, v1.y), h3 = __floats2bfloat162_rn(v1.z, v1.w);
          const uint4 val = make_uint4(*reinterpret_cast<uint32_t*>(&h0), *reinterpret_cast<uint32_t*>(&h1),
                                       *reinterpret_cast<uint32_t*>(&h2), *reinterpret_cast<uint32_t*>(&h3));
          const int row_r = __shfl_sync(0xffffffffu, row, r);
          if (row_r >= 0 && FMOE_ROW_OK(p, row_r)) {
            __nv_bfloat16* drow = p.row_ptrs
                ? reinterpret_cast<__nv_bfloat16*>(p.row_ptrs[row_r]) + n_blk * kTileN
                : hbase + static_cast<size_t>(row_r) * p.ld_out;
            *reinterpret_cast<uint4*>(drow + c * 32 + seg * 8) = val;
          }
        }
      } else {
        // 8 lanes per row, 4 rows per store instruction: 128 contiguous bytes per row
#pragma unroll
        for (int it = 0; it < 8; ++it) {
          const int r = it * 4 + (lane >> 3);
          const int seg = lane & 7;
          const float4 val = *reinterpret_cast<const float4*>(stage + r * kStageWordsPerRow + seg * 4);
          const int row_r = __shfl_sync(0xffffffffu, row, r);
          if (row_r >= 0 && FMOE_ROW_OK(p, row_r))
            *reinterpret_cast<float4*>(obase + static_cast<size_t>(row_r) * p.ld_out + c * 32 + seg * 4) = val;
        }
      }
    }
  }
}

// kARows: rows of the A tile that are actually fetched per K stage.  128 is the general
// case.  For decode-sized batches (at most kARows routed rows in total, hence per expert) only
// the first kARows rows of a block are real, so only those are loaded: the stage shrinks to
// kARows*128 + 32 KiB bytes, one more stage fits, and more weight bytes are in flight per SM.
// The MMA still reads 128 rows; the rows past kARows alias the start of the B slab, produce
// values that belong to pad slots only, and are never stored.
constexpr int kDecodeARows = 32;

template <int kARows> struct GemmStageCfg {
  static constexpr int kAStageBytes = kARows * kStageKBytes;
  static constexpr int kStageBytesT = kAStageBytes + kBBytes;
  static constexpr int kStagesT = kARows == kBlockM ? kStages : 5;
  static constexpr int kSmemBytesT = kStagesT * kStageBytesT + kSmemMisc + kEpiStageReserve + 1024;
};

template <bool kFp8, int kEpi, int kARows = kBlockM>
__global__ void __launch_bounds__(kGemmThreads, 1)
fmoe_grouped_gemm_kernel(const __grid_constant__ CUtensorMap tm_a,
                         const __grid_constant__ CUtensorMap tm_b, const GemmParams p) {
  using Cfg = GemmStageCfg<kARows>;
  constexpr int kStages = Cfg::kStagesT;             // shadows the general-case constants
  constexpr int kStageBytes = Cfg::kStageBytesT;
  constexpr int kABytes = Cfg::kAStageBytes;
  extern __shared__ uint8_t smem_raw[];
  // 128-byte-swizzled tiles need 1024-byte alignment.
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* misc = smem + kStages * kStageBytes;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(misc);            // [kStages]
  uint64_t* empty_bar = full_bar + kStages;                          // [kStages]
  uint64_t* acc_full_bar = empty_bar + kStages;                      // [2]
  uint64_t* acc_empty_bar = acc_full_bar + 2;                        // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty_bar + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  int* cum_s = reinterpret_cast<int*>(misc + 256);                   // [E + 1] copy of mblk_cum

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  constexpr int kElemsPerStage = kFp8 ? 128 : 64;   // K elements per stage
  constexpr int kUmmaKBytes = 32;                   // one MMA consumes 32 bytes of K per row

  // Set-up that needs nothing from the previous kernel on the stream runs before the
  // dependency wait, so under programmatic dependent launch it overlaps that kernel's tail.
  if (threadIdx.x == 0) {
    ptx::prefetch_tensormap(&tm_a);
    ptx::prefetch_tensormap(&tm_b);
    for (int s = 0; s < kStages; ++s) {
      ptx::mbar_init(ptx::smem_u32(&full_bar[s]), 1);
      ptx::mbar_init(ptx::smem_u32(&empty_bar[s]), 1);
    }
    for (int b = 0; b < 2; ++b) {
      ptx::mbar_init(ptx::smem_u32(&acc_full_bar[b]), 1);
      ptx::mbar_init(ptx::smem_u32(&acc_empty_bar[b]), 128);
    }
    *abort_flag = 0;
    ptx::fence_barrier_init();
    ptx::fence_proxy_async();
  }
  if (warp == 1) {
    ptx::tmem_alloc(ptx::smem_u32(tmem_slot), kTmemCols);
    ptx::tmem_relinquish();
  }
  // Everything the previous kernel produced is read after this point.
  ptx::pdl_wait();
  // The block table is read on every tile boundary by the producer; keep it on chip so the
  // decode does not sit on the critical path with dependent global loads.
  for (int i = threadIdx.x; i <= p.num_experts; i += kGemmThreads) cum_s[i] = p.mblk_cum[i];
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int total_tiles = cum_s[p.num_experts] * p.n_blocks;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x) {
        const TileCoord tc = decode_tile(tile, cum_s, p.num_experts, p.n_blocks);
        const int a_row = tc.m_blk * kBlockM;
        const int b_row0 = tc.expert * p.b_rows_per_expert + tc.n_blk * p.n_stride;
        const int b_row1 = b_row0 + p.second_slab_offset;
        for (int k = 0; k < p.k_iters; ++k) {
          if (!ptx::mbar_wait(ptx::smem_u32(&empty_bar[stage]), phase ^ 1u, abort_flag)) {
            ok = false;
            break;
          }
          const uint32_t full = ptx::smem_u32(&full_bar[stage]);
          const uint32_t sa = ptx::smem_u32(smem + stage * kStageBytes);
          const uint32_t sb = sa + kABytes;
          ptx::mbar_arrive_expect_tx(full, kStageBytes);
          const int kx = k * kElemsPerStage;
          int bx, by0, by1;
          b_coords(p, b_row0, k, kElemsPerStage, bx, by0);
          b_coords(p, b_row1, k, kElemsPerStage, bx, by1);
          ptx::tma_load_2d(sa, &tm_a, full, kx, a_row);
          ptx::tma_load_2d(sb, &tm_b, full, bx, by0);
          ptx::tma_load_2d(sb + kSlabRows * kStageKBytes, &tm_b, full, bx, by1);
          if (++stage == kStages) { stage = 0; phase ^= 1u; }
        }
      }
      if (!ok) atomicExch(p.status, kStatusGemmTimeout | 1);
      // every operand of this CTA has been requested: the next kernel on the stream may start
      // its own set-up while the last tiles are multiplied and stored
      ptx::pdl_release();
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x) {
        if (!ptx::mbar_wait(ptx::smem_u32(&acc_empty_bar[acc]), acc_phase ^ 1u, abort_flag)) {
          ok = false;
          break;
        }
        ptx::tc_fence_after();
        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * kTileN);
        for (int k = 0; k < p.k_iters; ++k) {
          if (!ptx::mbar_wait(ptx::smem_u32(&full_bar[stage]), phase, abort_flag)) {
            ok = false;
            break;
          }
          ptx::tc_fence_after();
          const uint32_t sa = ptx::smem_u32(smem + stage * kStageBytes);
          const uint64_t da = ptx::make_smem_desc(p.desc_template, sa);
          const uint64_t db = ptx::make_smem_desc(p.desc_template, sa + kABytes);
#pragma unroll
          for (int kk = 0; kk < kStageKBytes / kUmmaKBytes; ++kk) {
            // advancing K inside the swizzle row = advancing the start address
            const uint64_t adv = static_cast<uint64_t>((kk * kUmmaKBytes) >> 4);
            const uint32_t accum = (k | kk) ? 1u : 0u;
            if (FMOE_DBG(p, 2u)) continue;
            if (kFp8) ptx::umma_f8(d_tmem, da + adv, db + adv, p.idesc, accum);
            else      ptx::umma_f16(d_tmem, da + adv, db + adv, p.idesc, accum);
          }
          ptx::umma_commit(ptx::smem_u32(&empty_bar[stage]));   // frees the stage when MMAs finish
          if (++stage == kStages) { stage = 0; phase ^= 1u; }
        }
        if (!ok) break;
        ptx::umma_commit(ptx::smem_u32(&acc_full_bar[acc]));    // accumulator ready
        if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
      }
      if (!ok) atomicExch(p.status, kStatusGemmTimeout | 2);
    }
  } else {
    // ------------------------------------------------------------------ epilogue warps
    const int quad = warp & 3;                       // TMEM lane quadrant this warp may read
    const int epi_tid = threadIdx.x - 64;            // 0..127
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x) {
      const TileCoord tc = decode_tile(tile, cum_s, p.num_experts, p.n_blocks);
      const int b_row0 = tc.expert * p.b_rows_per_expert + tc.n_blk * p.n_stride;
      // Per-output-channel scales of this tile's two slabs (same addresses for the whole
      // warp, so these are broadcast loads served by L1).
      const float* bs0 = p.b_scale ? p.b_scale + b_row0 : nullptr;
      const float* bs1 = p.b_scale ? bs0 + p.second_slab_offset : nullptr;
      const int slot = tc.m_blk * kBlockM + quad * 32 + lane;   // sorted slot of this thread's row
      const float a_s = p.a_scale ? p.a_scale[slot] : 1.0f;
      if (!ptx::mbar_wait(ptx::smem_u32(&acc_full_bar[acc]), acc_phase, abort_flag)) {
        ok = false;
        break;
      }
      ptx::tc_fence_after();
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) +
                             static_cast<uint32_t>(acc * kTileN);
      if (!FMOE_DBG(p, 1u))
        epilogue_tile<kEpi>(p, t_row, slot, tc.n_blk, bs0, bs1, a_s,
                            reinterpret_cast<uint32_t*>(misc + kSmemMisc) + quad * (kEpiStageBytesPerWarp / 4));
      ptx::tc_fence_before();
      ptx::mbar_arrive(ptx::smem_u32(&acc_empty_bar[acc]));
      if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
    }
    if (!ok && epi_tid == 0) atomicExch(p.status, kStatusGemmTimeout | 3);
  }

  ptx::tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc(tmem_base, kTmemCols);
  }
  if (kEpi == kEpiScaledSlots) grid_done_signal(p);
}

// ============================================================================= CTA-pair variant
// Two CTAs of a cluster (two SMs) compute one 256-row x 256-column tile with
// tcgen05.mma.cta_group::2: CTA rank r stages the A rows of row block (2*pair + r) and the
// r-th 128-row slab of B (gate slab / up slab for the first GEMM), so every SM fetches half as
// much of the weight operand per flop as the single-CTA kernel.  Rank 0 issues the MMAs for
// both SMs; each CTA's tensor memory receives its own 128 accumulator rows and runs its own
// epilogue.  An expert with an odd number of row blocks leaves the second half of its last
// pair without rows: that half computes on whatever the next block holds and skips its
// epilogue.
constexpr int kPairStages = 6;
constexpr int kPairStageBytes = kABytes + kSlabRows * kStageKBytes;   // 16 KiB A + 16 KiB B slab
constexpr int kPairSmemMisc = 9216;                                   // barriers + two expert tables
constexpr int kPairSmemBytes = kPairStages * kPairStageBytes + kPairSmemMisc + kEpiStageReserve + 1024;

struct PairTile {
  int expert, n_blk, m_blk0, m_end;   // m_blk0: first row block of the pair; m_end: expert's end
};

__device__ __forceinline__ PairTile decode_pair_tile(int tile, const int* cum, const int* pair_cum,
                                                     int E, int n_blocks) {
  int lo = 1, hi = E;
  while (lo < hi) {
    int mid = (lo + hi) >> 1;
    if (pair_cum[mid] * n_blocks > tile) hi = mid; else lo = mid + 1;
  }
  PairTile t;
  t.expert = lo - 1;
  const int pbase = pair_cum[t.expert];
  const int pcnt = pair_cum[t.expert + 1] - pbase;
  const int local = tile - pbase * n_blocks;
  t.n_blk = local / pcnt;
  t.m_blk0 = cum[t.expert] + 2 * (local % pcnt);
  t.m_end = cum[t.expert + 1];
  return t;
}

template <bool kFp8, int kEpi>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kGemmThreads, 1)
fmoe_grouped_gemm_pair_kernel(const __grid_constant__ CUtensorMap tm_a,
                              const __grid_constant__ CUtensorMap tm_b, const GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* misc = smem + kPairStages * kPairStageBytes;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(misc);            // [kPairStages] used in rank 0
  uint64_t* empty_bar = full_bar + kPairStages;                      // [kPairStages] both ranks
  uint64_t* acc_full_bar = empty_bar + kPairStages;                  // [2] both ranks
  uint64_t* acc_empty_bar = acc_full_bar + 2;                        // [2] used in rank 0
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty_bar + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  int* cum_s = reinterpret_cast<int*>(misc + 256);                   // [E + 1]
  int* pair_cum_s = cum_s + 1032;                                    // [E + 1]

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = ptx::cluster_ctarank();
  constexpr int kElemsPerStage = kFp8 ? 128 : 64;
  constexpr int kUmmaKBytes = 32;

  if (threadIdx.x == 0) {
    ptx::prefetch_tensormap(&tm_a);
    ptx::prefetch_tensormap(&tm_b);
    for (int s = 0; s < kPairStages; ++s) {
      ptx::mbar_init(ptx::smem_u32(&full_bar[s]), 1);
      ptx::mbar_init(ptx::smem_u32(&empty_bar[s]), 1);
    }
    for (int b = 0; b < 2; ++b) {
      ptx::mbar_init(ptx::smem_u32(&acc_full_bar[b]), 1);
      ptx::mbar_init(ptx::smem_u32(&acc_empty_bar[b]), 8);     // 4 epilogue warps in each CTA
    }
    *abort_flag = 0;
    ptx::fence_barrier_init();
    ptx::fence_proxy_async();
  }
  if (warp == 1) {
    ptx::tmem_alloc_pair(ptx::smem_u32(tmem_slot), kTmemCols);
    ptx::tmem_relinquish_pair();
  }
  // set-up above needs nothing from the previous kernel; its output is read from here on
  ptx::pdl_wait();
  for (int i = threadIdx.x; i <= p.num_experts; i += kGemmThreads) cum_s[i] = p.mblk_cum[i];
  __syncthreads();
  if (threadIdx.x == 0) {
    int run = 0;
    pair_cum_s[0] = 0;
    for (int e = 0; e < p.num_experts; ++e) {
      run += (cum_s[e + 1] - cum_s[e] + 1) >> 1;
      pair_cum_s[e + 1] = run;
    }
  }
  ptx::tc_fence_before();
  ptx::cluster_sync_all();      // barriers of both CTAs are initialised before anyone signals them
  ptx::tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int total_tiles = pair_cum_s[p.num_experts] * p.n_blocks;
  const int first_tile = blockIdx.x >> 1;
  const int tile_step = gridDim.x >> 1;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer (both ranks)
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = first_tile; ok && tile < total_tiles; tile += tile_step) {
        const PairTile tc = decode_pair_tile(tile, cum_s, pair_cum_s, p.num_experts, p.n_blocks);
        const int a_row = (tc.m_blk0 + static_cast<int>(rank)) * kBlockM;
        const int b_row = tc.expert * p.b_rows_per_expert + tc.n_blk * p.n_stride +
                          (rank ? p.second_slab_offset : 0);
        for (int k = 0; k < p.k_iters; ++k) {
          if (!ptx::mbar_wait(ptx::smem_u32(&empty_bar[stage]), phase ^ 1u, abort_flag)) {
            ok = false;
            break;
          }
          // completion bytes of both CTAs are credited to rank 0's barrier
          const uint32_t full0 = ptx::map_to_rank(ptx::smem_u32(&full_bar[stage]), 0);
          const uint32_t sa = ptx::smem_u32(smem + stage * kPairStageBytes);
          if (rank == 0) ptx::mbar_arrive_expect_tx(ptx::smem_u32(&full_bar[stage]), 2 * kPairStageBytes);
          const int kx = k * kElemsPerStage;
          int bx, by;
          b_coords(p, b_row, k, kElemsPerStage, bx, by);
          ptx::tma_load_2d_pair(sa, &tm_a, full0, kx, a_row);
          ptx::tma_load_2d_pair(sa + kABytes, &tm_b, full0, bx, by);
          if (++stage == kPairStages) { stage = 0; phase ^= 1u; }
        }
      }
      if (!ok) atomicExch(p.status, kStatusGemmTimeout | 0x11);
      ptx::pdl_release();   // all operands requested: the next kernel may begin its set-up
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer (rank 0 only)
    if (lane == 0 && rank == 0) {
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int tile = first_tile; ok && tile < total_tiles; tile += tile_step) {
        if (!ptx::mbar_wait(ptx::smem_u32(&acc_empty_bar[acc]), acc_phase ^ 1u, abort_flag)) {
          ok = false;
          break;
        }
        ptx::tc_fence_after();
        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * kTileN);
        for (int k = 0; k < p.k_iters; ++k) {
          if (!ptx::mbar_wait(ptx::smem_u32(&full_bar[stage]), phase, abort_flag)) {
            ok = false;
            break;
          }
          ptx::tc_fence_after();
          const uint32_t sa = ptx::smem_u32(smem + stage * kPairStageBytes);
          const uint64_t da = ptx::make_smem_desc(p.desc_template, sa);
          const uint64_t db = ptx::make_smem_desc(p.desc_template, sa + kABytes);
#pragma unroll
          for (int kk = 0; kk < kStageKBytes / kUmmaKBytes; ++kk) {
            const uint64_t adv = static_cast<uint64_t>((kk * kUmmaKBytes) >> 4);
            const uint32_t accum = (k | kk) ? 1u : 0u;
            if (FMOE_DBG(p, 2u)) continue;
            if (kFp8) ptx::umma_f8_pair(d_tmem, da + adv, db + adv, p.idesc, accum);
            else      ptx::umma_f16_pair(d_tmem, da + adv, db + adv, p.idesc, accum);
          }
          // the stage is free in both CTAs once these MMAs have read it
          const uint32_t e_local = ptx::smem_u32(&empty_bar[stage]);
          ptx::umma_commit_pair(e_local);
          ptx::umma_commit_pair(ptx::map_to_rank(e_local, 1));
          if (++stage == kPairStages) { stage = 0; phase ^= 1u; }
        }
        if (!ok) break;
        const uint32_t f_local = ptx::smem_u32(&acc_full_bar[acc]);
        ptx::umma_commit_pair(f_local);
        ptx::umma_commit_pair(ptx::map_to_rank(f_local, 1));
        if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
      }
      if (!ok) atomicExch(p.status, kStatusGemmTimeout | 0x12);
    }
  } else {
    // ------------------------------------------------------------------ epilogue warps (both ranks)
    const int quad = warp & 3;
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    for (int tile = first_tile; ok && tile < total_tiles; tile += tile_step) {
      const PairTile tc = decode_pair_tile(tile, cum_s, pair_cum_s, p.num_experts, p.n_blocks);
      const int m_blk = tc.m_blk0 + static_cast<int>(rank);
      const bool valid = m_blk < tc.m_end;
      const int b_row0 = tc.expert * p.b_rows_per_expert + tc.n_blk * p.n_stride;
      const float* bs0 = p.b_scale ? p.b_scale + b_row0 : nullptr;
      const float* bs1 = p.b_scale ? bs0 + p.second_slab_offset : nullptr;
      const int slot = m_blk * kBlockM + quad * 32 + lane;
      const float a_s = (p.a_scale && valid) ? p.a_scale[slot] : 1.0f;
      if (!ptx::mbar_wait(ptx::smem_u32(&acc_full_bar[acc]), acc_phase, abort_flag)) {
        ok = false;
        break;
      }
      ptx::tc_fence_after();
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) +
                             static_cast<uint32_t>(acc * kTileN);
      if (valid && !FMOE_DBG(p, 1u))
        epilogue_tile<kEpi>(p, t_row, slot, tc.n_blk, bs0, bs1, a_s,
                            reinterpret_cast<uint32_t*>(misc + kPairSmemMisc) + quad * (kEpiStageBytesPerWarp / 4));
      ptx::tc_fence_before();
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive_cluster(ptx::map_to_rank(ptx::smem_u32(&acc_empty_bar[acc]), 0));
      if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
    }
    if (!ok && threadIdx.x == 64) atomicExch(p.status, kStatusGemmTimeout | 0x13);
  }

  // Neither CTA may leave while its partner can still signal its barriers or read its
  // shared memory through a pair MMA.
  ptx::tc_fence_before();
  ptx::cluster_sync_all();
  if (warp == 1) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc_pair(tmem_base, kTmemCols);
  }
  if (kEpi == kEpiScaledSlots) grid_done_signal(p);
}

}  // namespace fmoe
