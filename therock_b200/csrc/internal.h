// Launchers shared between the translation units of libfmoe_b200.so (not part of the ABI).
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace fmoe {

// Launch `kernel` allowing it to overlap the tail of the previous kernel on the stream
// (programmatic dependent launch).  The kernel must execute griddepcontrol.wait before it
// touches its predecessor's output.  FMOE_PDL=0 turns the attribute off.
bool pdl_enabled();
template <typename... KArgs, typename... Args>
cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                       Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = pdl_enabled() ? 1 : 0;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// moe_sorting.  All outputs are device pointers; sorted_rows, mblk_cum and status_to_clear
// (a status word the kernel resets to 0) may be null.  num_tokens_dev (optional) is a device
// int that lowers the token count below T; id_div > 1 buckets by id / id_div (the rank
// that owns the expert); inv_out[T*K] receives each pair's slot (-1 if dropped); scratch
// (sort_scratch_words(E) ints, with mblk_cum) enables the multi-CTA path for >= 8192 pairs.
cudaError_t launch_moe_sorting(const int32_t* topk_ids, const float* topk_weight, int T, int K,
                               int E, int block_m, int64_t cap, int32_t* sorted_token_ids,
                               float* sorted_weights, int32_t* sorted_rows,
                               int32_t* sorted_expert_ids, int32_t* num_post_pad,
                               int32_t* mblk_cum, int32_t* status_to_clear, cudaStream_t stream,
                               const int32_t* num_tokens_dev = nullptr, int id_div = 1,
                               int32_t* inv_out = nullptr, int32_t* scratch = nullptr);
// int32 words of `scratch` that lets launch_moe_sorting spread large inputs over several CTAs.
constexpr size_t sort_scratch_words(int E) { return 2 * 64 * static_cast<size_t>(E); }

// Gather rows of a bf16 matrix into sorted order, optionally quantising each row to e4m3.
//   src [n_src, cols] bf16; row_ids [cap] (entry >= n_src means pad -> zero row) or null
//   for identity; only slots < *num_post_pad are touched.
//   quant 0: dst bf16 [cap, cols].  quant 1: dst e4m3 [cap, cols] + scales[cap] (one per
//   row).  quant 2: dst e4m3 + scales [cap, cols/128] (one per 128 columns).
//   live_ids (optional, [cap]): slots whose entry is negative are skipped entirely.
cudaError_t launch_gather_rows(const void* src, int n_src, int cols, const int32_t* row_ids,
                               const int32_t* num_post_pad, int64_t cap, int quant, void* dst,
                               float* scales, cudaStream_t stream, const int32_t* live_ids = nullptr);

// out[t, :] = bf16( sum_k slots[t*K + k, :] ) over the k whose expert id lies in [0, E).
cudaError_t launch_combine(const float* slots, const int32_t* topk_ids, int T, int K, int E,
                           int H, void* out, cudaStream_t stream,
                           const int32_t* num_tokens_dev = nullptr);

// out[t, :] = bf16( sum_k rows[index[t*K + k], :] ), f32 accumulation, index < 0 skipped;
// rows are bf16 [*, H].
cudaError_t launch_combine_rows(const void* rows, const int32_t* index, int T, int K, int H,
                                void* out, cudaStream_t stream);

struct GemmLaunch {
  bool fp8;
  int epilogue;                 // kEpiSiluMul / kEpiScaledSlots
  const void* a;                // [a_rows, k_elems] row-major
  int64_t a_rows;
  const void* b;                // [E * b_rows_per_expert, k_elems] row-major
  int k_elems;
  int num_experts;
  int b_rows_per_expert;
  int n_blocks, n_stride, second_slab_offset;
  const int32_t* mblk_cum;
  const int32_t* sorted_rows;
  const float* sorted_weights;
  const float* a_scale;
  const float* b_scale;
  void* out;
  int ld_out;
  int32_t* status;
  int max_m_blocks;             // upper bound on 128-row blocks (sizes the grid)
  int max_live_rows;            // upper bound on real rows in any block (0 = unknown, i.e. 128)
  bool b_tiled;                 // B is stored as contiguous 128-row x 128-byte tiles (see fmoe_weight_layout)
  bool block_scale;             // fp8 with 1x128 activation groups and 128x128 weight blocks:
                                // a_scale is [a_rows, K/128], b_scale [E*b_rows/128, K/128]
  int mode;                     // 2 = CTA-pair kernel (cta_group::2), anything else = single-CTA kernel
  uint64_t desc_template_override;  // 0 = the library's descriptor encoding (diagnostics only)
  uint32_t idesc_override;          // 0 = the library's instruction descriptor
};
// Returns cudaSuccess or the failing CUDA error; *drv_err receives a CUresult when the
// tensor-map encode fails.
cudaError_t launch_grouped_gemm(const GemmLaunch& g, cudaStream_t stream, int* drv_err);

// 0 = no override, 1 / 2 = FMOE_GEMM_MODE forces the single-CTA / CTA-pair kernel.
int gemm_mode_from_env();
// SM count of the current device (cached).
int device_sm_count();

}  // namespace fmoe
