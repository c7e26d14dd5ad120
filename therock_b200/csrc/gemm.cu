// Host side of the grouped GEMM: TMA descriptors and the persistent launch.
#include <cuda.h>

#include <cstdlib>
#include <cstring>
#include <mutex>

#include "../../include/fused_moe_c.h"
#include "gemm_tokn.cuh"
#include "internal.h"

namespace fmoe {
namespace {

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                   const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                   const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// The driver entry point is looked up through the runtime so the library does not link
// libcuda directly.
EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

// Row-major [rows, k_elems] matrix, box = 128 bytes of K x box_rows rows, 128-byte swizzle.
CUresult make_map(CUtensorMap* tm, const void* base, bool fp8, int64_t rows, int k_elems,
                  int box_rows = kSlabRows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return CUDA_ERROR_NOT_FOUND;
  const int esize = fp8 ? 1 : 2;
  cuuint64_t dims[2] = {static_cast<cuuint64_t>(k_elems), static_cast<cuuint64_t>(rows)};
  cuuint64_t strides[1] = {static_cast<cuuint64_t>(k_elems) * esize};
  cuuint32_t box[2] = {static_cast<cuuint32_t>(kStageKBytes / esize), static_cast<cuuint32_t>(box_rows)};
  cuuint32_t estr[2] = {1, 1};
  return fn(tm, fp8 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2,
            const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
            CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
}

constexpr int kMaxDevices = 64;

int current_device() {
  int dev = 0;
  cudaGetDevice(&dev);
  return (dev >= 0 && dev < kMaxDevices) ? dev : 0;
}

int sm_count() {
  static int n[kMaxDevices] = {0};
  const int dev = current_device();
  if (n[dev] == 0) {
    int v = 0;
    cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev);
    n[dev] = v > 0 ? v : 148;
  }
  return n[dev];
}

template <bool kFp8, int kEpi, int kARows = kBlockM>
cudaError_t launch_variant(const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p,
                           int grid, cudaStream_t stream) {
  static bool configured[kMaxDevices] = {false};   // per instantiation and device
  constexpr int kSmem = GemmStageCfg<kARows>::kSmemBytesT;
  const int dev = current_device();
  if (!configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(fmoe_grouped_gemm_kernel<kFp8, kEpi, kARows>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem);
    if (e != cudaSuccess) return e;
    configured[dev] = true;
  }
  return launch_pdl(fmoe_grouped_gemm_kernel<kFp8, kEpi, kARows>, dim3(grid), dim3(kGemmThreads), kSmem, stream,
                    ta, tb, p);
}

template <bool kFp8, int kEpi>
cudaError_t launch_pair_variant(const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p,
                                int grid, cudaStream_t stream) {
  static bool configured[kMaxDevices] = {false};
  const int dev = current_device();
  if (!configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(fmoe_grouped_gemm_pair_kernel<kFp8, kEpi>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, kPairSmemBytes);
    if (e != cudaSuccess) return e;
    configured[dev] = true;
  }
  return launch_pdl(fmoe_grouped_gemm_pair_kernel<kFp8, kEpi>, dim3(grid), dim3(kGemmThreads), kPairSmemBytes,
                    stream, ta, tb, p);
}

}  // namespace

// A library built with -DFMOE_TIMING_SWITCHES honours FMOE_GEMM_MODE=1cta / 2cta, which forces one
// kernel flavour for every GEMM (used to compare them); the product build ignores the variable.
int gemm_mode_override() {
#ifdef FMOE_TIMING_SWITCHES
  static int mode = -1;
  if (mode < 0) {
    const char* e = getenv("FMOE_GEMM_MODE");
    mode = !e ? 0 : (std::strcmp(e, "1cta") == 0 ? 1 : (std::strcmp(e, "2cta") == 0 ? 2 : 0));
  }
  return mode;
#else
  return 0;
#endif
}

int device_sm_count() { return sm_count(); }

bool pdl_enabled() {
  static int on = -1;
  if (on < 0) {
    const char* e = getenv("FMOE_PDL");
    on = (e && std::strcmp(e, "0") == 0) ? 0 : 1;
  }
  return on == 1;
}

template <int kEpi, bool kHw, int kNT = kTileN>
cudaError_t launch_block_variant(const CUtensorMap& ta, const CUtensorMap& tb, const BlockGemmParams& bp, int grid,
                                 cudaStream_t stream) {
  static bool configured[kMaxDevices] = {false};
  const int dev = current_device();
  if (!configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(fmoe_grouped_gemm_block_kernel<kEpi, kHw, kNT>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, kBlockSmemBytes);
    if (e != cudaSuccess) return e;
    configured[dev] = true;
  }
  return launch_pdl(fmoe_grouped_gemm_block_kernel<kEpi, kHw, kNT>, dim3(grid), dim3(kBlockGemmThreads),
                    kBlockSmemBytes, stream, ta, tb, bp);
}

template <int kEpi>
cudaError_t launch_tokn_variant(const CUtensorMap& tw, const CUtensorMap (&tt)[4], const BlockGemmParams& bp, int grid,
                                cudaStream_t stream) {
  static bool configured[kMaxDevices] = {false};
  const int dev = current_device();
  if (!configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(fmoe_grouped_gemm_tokn_kernel<kEpi>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, kToknSmemBytes);
    if (e != cudaSuccess) return e;
    configured[dev] = true;
  }
  return launch_pdl(fmoe_grouped_gemm_tokn_kernel<kEpi>, dim3(grid), dim3(kToknThreads), kToknSmemBytes, stream, tw,
                    tt[0], tt[1], tt[2], tt[3], bp);
}

cudaError_t launch_grouped_gemm(const GemmLaunch& g, cudaStream_t stream, int* drv_err) {
  CUtensorMap ta, tb;
  const bool tokn = g.flavour == FMOE_KERNEL_BLOCK_HW_TOKENS_N;
  const bool block = g.flavour == FMOE_KERNEL_BLOCK_PROMOTE || g.flavour == FMOE_KERNEL_BLOCK_HW_SCALE || tokn;
  const bool pair = g.flavour == FMOE_KERNEL_PAIR;
  // decode-sized batches: only the first kDecodeARows rows of a block can be real
  const bool few_rows = g.flavour == FMOE_KERNEL_SINGLE_DECODE;
  CUresult r = make_map(&ta, g.a, g.fp8, g.a_rows, g.k_elems, few_rows ? kDecodeARows : kSlabRows);
  const int esize = g.fp8 ? 1 : 2;
  const int k_blocks = (g.k_elems * esize + kStageKBytes - 1) / kStageKBytes;
  if (r == CUDA_SUCCESS) {
    if (g.b_tiled)   // a [tiles * 128, 128 bytes] matrix: every box is one contiguous 16 KiB tile
      r = make_map(&tb, g.b, g.fp8, static_cast<int64_t>(g.num_experts) * g.b_rows_per_expert * k_blocks,
                   kStageKBytes / esize);
    else
      r = make_map(&tb, g.b, g.fp8, static_cast<int64_t>(g.num_experts) * g.b_rows_per_expert, g.k_elems);
  }
  if (r != CUDA_SUCCESS) {
    if (drv_err) *drv_err = static_cast<int>(r);
    return cudaErrorInvalidValue;
  }
  GemmParams p{};
  p.mblk_cum = g.mblk_cum;
  p.num_experts = g.num_experts;
  p.n_blocks = g.n_blocks;
  p.k_iters = k_blocks;
  p.b_rows_per_expert = g.b_rows_per_expert;
  p.n_stride = g.n_stride;
  p.second_slab_offset = g.second_slab_offset;
  p.sorted_rows = g.sorted_rows;
  p.sorted_weights = g.sorted_weights;
  p.a_scale = static_cast<const float*>(g.a_scale);
  p.b_scale = g.b_scale;
  p.out = g.out;
  p.ld_out = g.ld_out;
  p.out_bf16 = g.out_bf16 ? 1 : 0;
  p.out_rows = g.out_rows;
  p.row_ptrs = g.row_ptrs;
  p.done_addrs = g.done_addrs;
  p.done_value = g.done_value;
  p.done_counter = g.done_counter;
  p.done_count = g.done_count;
  p.status = g.status;
  p.b_tiled_kb = g.b_tiled ? k_blocks : 0;
#ifdef FMOE_TIMING_SWITCHES
  {
    static int dbg = -1;       // FMOE_DEBUG_FLAGS: timing experiments only
    if (dbg < 0) { const char* e = getenv("FMOE_DEBUG_FLAGS"); dbg = e ? atoi(e) : 0; }
    p.debug_flags = static_cast<uint32_t>(dbg);
  }
#endif
  p.desc_template = ptx::sw128_kmajor_desc_template();
  p.idesc = ptx::make_idesc(g.fp8 ? 0u : 1u, kBlockM, kTileN);
  const long long max_tiles = static_cast<long long>(g.max_m_blocks) * g.n_blocks;
  const int grid = static_cast<int>(max_tiles < sm_count() ? (max_tiles > 0 ? max_tiles : 1) : sm_count());
  if (block) {
    BlockGemmParams bp;
    bp.g = p;
    bp.g.a_scale = nullptr;
    bp.g.b_scale = nullptr;
    bp.a_scale = g.a_scale;
    bp.b_scale = g.b_scale;
    bp.k_blocks = p.k_iters;
    bp.a_rows = g.a_rows;
    bp.out_scale = g.out_scale;
    if (tokn) {
      if (g.epilogue == kEpiSilu) return cudaErrorInvalidValue;
      if (g.epilogue == kEpiSiluMul && g.out_scale == nullptr) return cudaErrorInvalidValue;
      // token boxes of 128, 64, 32 and 16 rows: every chunk (a multiple of 16 rows) is at most three loads
      CUtensorMap tt[4];
      const int box_rows[4] = {128, 64, 32, 16};
      for (int i = 0; i < 4; ++i) {
        CUresult r2 = make_map(&tt[i], g.a, true, g.a_rows, g.k_elems, box_rows[i]);
        if (r2 != CUDA_SUCCESS) {
          if (drv_err) *drv_err = static_cast<int>(r2);
          return cudaErrorInvalidValue;
        }
      }
      // upper bound on chunks: one per expert that is hit, plus one per full 224 rows
      const long long rows_bound = static_cast<long long>(g.max_m_blocks) * kBlockM;
      const long long chunk_bound = rows_bound / kToknMaxN + g.num_experts;
      const long long tile_bound = chunk_bound * g.n_blocks;
      const int tgrid = static_cast<int>(tile_bound < sm_count() ? (tile_bound > 0 ? tile_bound : 1) : sm_count());
      return g.epilogue == kEpiSiluMul ? launch_tokn_variant<kEpiSiluMul>(tb, tt, bp, tgrid, stream)
                                       : launch_tokn_variant<kEpiScaledSlots>(tb, tt, bp, tgrid, stream);
    }
    const bool hw = g.flavour == FMOE_KERNEL_BLOCK_HW_SCALE;
    if (hw && g.epilogue == kEpiScaledSlots && !g.b_tiled && g.ld_out % 224 == 0 && g.n_stride == kTileN) {
      // Output width tiles by 224: two 224-column accumulators fit tensor memory beside the scale
      // buffers, so the drain of one tile overlaps the MMAs of the next.
      CUtensorMap tb224;
      CUresult r2 = make_map(&tb224, g.b, true, static_cast<int64_t>(g.num_experts) * g.b_rows_per_expert, g.k_elems, 112);
      if (r2 != CUDA_SUCCESS) {
        if (drv_err) *drv_err = static_cast<int>(r2);
        return cudaErrorInvalidValue;
      }
      bp.g.n_blocks = g.ld_out / 224;
      bp.g.n_stride = 224;
      bp.g.second_slab_offset = 112;
      const long long tiles224 = static_cast<long long>(g.max_m_blocks) * bp.g.n_blocks;
      const int grid224 = static_cast<int>(tiles224 < sm_count() ? (tiles224 > 0 ? tiles224 : 1) : sm_count());
      return launch_block_variant<kEpiScaledSlots, true, 224>(ta, tb224, bp, grid224, stream);
    }
    if (g.epilogue == kEpiSiluMul) {
      if (g.out_scale == nullptr) return cudaErrorInvalidValue;   // the first GEMM always quantises its output
      return hw ? launch_block_variant<kEpiSiluMul, true>(ta, tb, bp, grid, stream)
                : launch_block_variant<kEpiSiluMul, false>(ta, tb, bp, grid, stream);
    }
    return hw ? launch_block_variant<kEpiScaledSlots, true>(ta, tb, bp, grid, stream)
              : launch_block_variant<kEpiScaledSlots, false>(ta, tb, bp, grid, stream);
  }
#define FMOE_DISPATCH_EPI(LAUNCH, FP8, GRID, ...)                                                  \
  (g.epilogue == kEpiSiluMul ? LAUNCH<FP8, kEpiSiluMul __VA_ARGS__>(ta, tb, p, GRID, stream)       \
   : g.epilogue == kEpiSilu  ? LAUNCH<FP8, kEpiSilu __VA_ARGS__>(ta, tb, p, GRID, stream)          \
                             : LAUNCH<FP8, kEpiScaledSlots __VA_ARGS__>(ta, tb, p, GRID, stream))
  if (pair) {
    p.idesc = ptx::make_idesc(g.fp8 ? 0u : 1u, 2 * kBlockM, kTileN);
    // upper bound on pair tiles: every expert may add one half-empty pair
    const long long max_pairs = (static_cast<long long>(g.max_m_blocks) + g.num_experts + 1) / 2;
    const long long max_ptiles = max_pairs * g.n_blocks;
    const int clusters = sm_count() / 2;
    const int pgrid = 2 * static_cast<int>(max_ptiles < clusters ? (max_ptiles > 0 ? max_ptiles : 1) : clusters);
    return g.fp8 ? FMOE_DISPATCH_EPI(launch_pair_variant, true, pgrid) : FMOE_DISPATCH_EPI(launch_pair_variant, false, pgrid);
  }
#define FMOE_COMMA_DECODE , kDecodeARows
  if (few_rows)
    return g.fp8 ? FMOE_DISPATCH_EPI(launch_variant, true, grid, FMOE_COMMA_DECODE)
                 : FMOE_DISPATCH_EPI(launch_variant, false, grid, FMOE_COMMA_DECODE);
  return g.fp8 ? FMOE_DISPATCH_EPI(launch_variant, true, grid) : FMOE_DISPATCH_EPI(launch_variant, false, grid);
#undef FMOE_COMMA_DECODE
#undef FMOE_DISPATCH_EPI
}

}  // namespace fmoe
