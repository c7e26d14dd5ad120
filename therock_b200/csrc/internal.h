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
//   for identity; only slots < *num_post_pad are touched (num_post_pad null: all `cap` slots).
//   quant 0: dst bf16 [cap, cols].  quant 1: dst e4m3 [cap, cols] + scales[cap] (one per
//   row).  quant 2: dst e4m3 + scales [cap, cols/128] (one per 128 columns).
//   live_ids (optional, [cap]): slots whose entry is negative are skipped entirely.
//   skip_pad: pad slots (row id outside the source) are left unwritten instead of zero-filled.
cudaError_t launch_gather_rows(const void* src, int n_src, int cols, const int32_t* row_ids,
                               const int32_t* num_post_pad, int64_t cap, int quant, void* dst,
                               void* scales, cudaStream_t stream, const int32_t* live_ids = nullptr,
                               bool skip_pad = false);

// dst[slot] = src[row_ids[slot]] for rows that are already e4m3 with their scales (quant 1, 2, 3 as
// above); only slots < *num_post_pad with a valid row id are written.  cols must be a multiple of 16.
cudaError_t launch_gather_quantised(const void* src, const void* src_scale, int n_src, int cols,
                                    const int32_t* row_ids, const int32_t* num_post_pad, int64_t cap, int quant,
                                    void* dst, void* dst_scale, cudaStream_t stream);

// Decode-sized batches (T*K <= 128, bf16 or per-token-quantised activations): moe_sorting and the
// gather (+ quantisation) in one launch.  Pad slots of a_sorted are left unwritten.
bool decode_prologue_applies(int T, int K, int quant);
cudaError_t launch_decode_prologue(const int32_t* topk_ids, const float* topk_weight, int T, int K, int E, int64_t cap,
                                   const void* x, int H, int quant, int32_t* sorted_token_ids, float* sorted_weights,
                                   int32_t* sorted_rows, int32_t* sorted_expert_ids, int32_t* num_post_pad,
                                   int32_t* mblk_cum, int32_t* status_to_clear, void* a_sorted, float* a_scale,
                                   cudaStream_t stream, const int32_t* num_tokens_dev);

// out[t, :] = bf16( sum_k slots[t*K + k, :] ) over the k whose expert id lies in [0, E);
// slots are f32, or bf16 when slots_bf16.
cudaError_t launch_combine(const void* slots, bool slots_bf16, const int32_t* topk_ids, int T, int K, int E,
                           int H, void* out, cudaStream_t stream,
                           const int32_t* num_tokens_dev = nullptr);

// out[t, :] = bf16( sum_k rows[index[t*K + k], :] ), f32 accumulation, index < 0 skipped;
// rows are bf16 [*, H].
cudaError_t launch_combine_rows(const void* rows, const int32_t* index, int T, int K, int H,
                                void* out, cudaStream_t stream);

struct GemmLaunch {
  bool fp8;
  int epilogue;                 // kEpiSiluMul / kEpiScaledSlots / kEpiSilu
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
  const void* a_scale;          // f32 [a_rows] (per row), f32 [a_rows, K/128] (block promote) or the
                                // UE8M0 bytes (block_scale MMA)
  const float* b_scale;         // f32 [E * b_rows] or [E * b_rows / 128, K/128]
  void* out;
  int ld_out;
  int64_t out_rows;             // rows of `out` (bound used by the checked build)
  bool out_bf16;                // kEpiScaledSlots: weighted rows stored as bf16 instead of f32
  const uint64_t* row_ptrs;     // with out_bf16: destination address of each routed pair's row (nullptr = out + pair * ld_out)
  const uint64_t* done_addrs;   // completion signal written by the last CTA (nullptr = none)
  const int32_t* done_value;
  int32_t* done_counter;
  int done_count;
  void* out_scale;              // block flavours, first GEMM: when set, `out` receives e4m3 and this the
                                // 1x128 scales of the intermediate (f32 [a_rows, ld_out/128] or UE8M0 bytes)
  int32_t* status;
  int max_m_blocks;             // upper bound on 128-row blocks (sizes the grid)
  bool b_tiled;                 // B is stored as contiguous 128-row x 128-byte tiles (see fmoe_weight_layout)
  int flavour;                  // fmoe_gemm_kernel
};
// Returns cudaSuccess or the failing CUDA error; *drv_err receives a CUresult when the
// tensor-map encode fails.
cudaError_t launch_grouped_gemm(const GemmLaunch& g, cudaStream_t stream, int* drv_err);

// 0 = no override; 1 / 2 force the single-CTA / CTA-pair kernel.  Always 0 unless the library
// was built with -DFMOE_TIMING_SWITCHES (then FMOE_GEMM_MODE=1cta|2cta is honoured).
int gemm_mode_override();
// SM count of the current device (cached).
int device_sm_count();

}  // namespace fmoe
