// C++ host surface of the B200 fused-MoE operator: the same three names a ck_tile user
// writes -- fused_moe_traits, fused_moe_args, fused_moe(traits, args, stream) -- plus the
// separately callable moe_sorting, implemented as thin inline code over the C-ABI in
// fused_moe_c.h.
//
// The ck_tile originals live in Composable Kernel, which TheRock builds from the
// rocm-libraries submodule (math-libs/CMakeLists.txt:582-608); that submodule is empty
// in the reference checkout, so field-for-field compatibility with the upstream structs
// cannot be verified and is not claimed.  The fields here are what the operator needs:
// dtype strings select the variant (traits), pointers and dimensions describe one call
// (args).  The return convention follows the ck_tile host API: elapsed milliseconds when
// timing was requested, 0 otherwise, a negative value on error.
#pragma once

#include <cstdint>
#include <string>

#include "fused_moe_c.h"

struct fused_moe_traits {
  std::string prec_i = "bf16";   // activation input type: "bf16"
  std::string prec_w = "bf16";   // weight type: "bf16" or "fp8"
  std::string prec_o = "bf16";   // output type: "bf16"
  std::string quant = "none";    // "none" | "token_channel" | "block128" | "block128_ue8m0"
  std::string activation = "silu";
  int gate_only = 0;             // 0: gate and up rows packed as [2I, H]
  int block_m = 128;             // sorted M-block
  int gemm_mode = 0;             // 0 = per-GEMM choice, 1 = single-CTA kernel, 2 = CTA-pair kernel
  std::string weight_layout = "row_major";   // or "tiled128": weights pre-shuffled into 16 KiB tiles
  std::string partial_dtype = "f32";         // "f32" | "bf16": weighted expert outputs before the ordered sum
};

struct fused_moe_args {
  const void* a_ptr = nullptr;             // [T, H] activations (bf16)
  const void* g_ptr = nullptr;             // [E, 2I, H] gate+up weights
  const void* d_ptr = nullptr;             // [E, H, I] down weights
  const float* g_scale_ptr = nullptr;      // gate+up weight scales (fp8 variants)
  const float* d_scale_ptr = nullptr;      // down weight scales (fp8 variants)
  const int32_t* topk_ids_ptr = nullptr;   // [T, K]
  const float* topk_weight_ptr = nullptr;  // [T, K]
  void* o_ptr = nullptr;                   // [T, H] output (bf16)
  void* ws_ptr = nullptr;                  // workspace, fused_moe_get_workspace_size bytes
  uint64_t ws_bytes = 0;
  int num_tokens = 0;
  int hidden_size = 0;
  int intermediate_size = 0;   // per expert, I (W1 has 2I rows)
  int num_experts = 0;
  int topk = 0;
  const int32_t* num_tokens_dev_ptr = nullptr;  // optional device-side token count (<= num_tokens)
  int expected_tokens = 0;                      // its typical value (kernel choice hint), 0 = num_tokens
  const uint64_t* partial_row_ptrs = nullptr;   // optional [T*K] destinations of the weighted partial rows (bf16)
  const void* a_scale_ptr = nullptr;            // optional: a_ptr holds e4m3 rows and this their scales (fmoe_quantise_rows)
};

struct stream_config {
  void* stream_id = nullptr;   // cudaStream_t
  bool time_kernel = false;    // true: synchronise and return elapsed ms
};

namespace fmoe_detail {
inline int to_c(const fused_moe_traits& t, fmoe_traits_c* c) {
  *c = fmoe_traits_c{};
  if (t.prec_i != "bf16" || t.prec_o != "bf16") return FMOE_ERR_UNSUPPORTED;
  if (t.quant == "none") c->quant = FMOE_QUANT_NONE;
  else if (t.quant == "token_channel") c->quant = FMOE_QUANT_TOKEN_CHANNEL;
  else if (t.quant == "block128") c->quant = FMOE_QUANT_BLOCK128;
  else if (t.quant == "block128_ue8m0") c->quant = FMOE_QUANT_BLOCK128_UE8M0;
  else return FMOE_ERR_INVALID_ARG;
  if (t.prec_w == "bf16") c->weight_dtype = FMOE_BF16;
  else if (t.prec_w == "fp8") c->weight_dtype = FMOE_FP8_E4M3;
  else return FMOE_ERR_INVALID_ARG;
  if (t.activation != "silu") return FMOE_ERR_UNSUPPORTED;
  c->activation = FMOE_ACT_SILU;
  c->gate_only = t.gate_only;
  c->block_m = t.block_m;
  c->gemm_mode = t.gemm_mode;
  if (t.weight_layout == "row_major") c->weight_layout = FMOE_WEIGHTS_ROW_MAJOR;
  else if (t.weight_layout == "tiled128") c->weight_layout = FMOE_WEIGHTS_TILED128;
  else return FMOE_ERR_INVALID_ARG;
  if (t.partial_dtype == "f32") c->partial_dtype = FMOE_PARTIAL_F32;
  else if (t.partial_dtype == "bf16") c->partial_dtype = FMOE_PARTIAL_BF16;
  else return FMOE_ERR_INVALID_ARG;
  return FMOE_OK;
}
inline void to_c(const fused_moe_args& a, fmoe_args_c* c) {
  *c = fmoe_args_c{};
  c->x = a.a_ptr; c->w1 = a.g_ptr; c->w2 = a.d_ptr;
  c->w1_scale = a.g_scale_ptr; c->w2_scale = a.d_scale_ptr;
  c->topk_ids = a.topk_ids_ptr; c->topk_weight = a.topk_weight_ptr;
  c->out = a.o_ptr; c->workspace = a.ws_ptr; c->workspace_bytes = a.ws_bytes;
  c->T = a.num_tokens; c->H = a.hidden_size; c->I = a.intermediate_size;
  c->E = a.num_experts; c->K = a.topk;
  c->num_tokens_dev = a.num_tokens_dev_ptr;
  c->expected_tokens = a.expected_tokens;
  c->partial_row_ptrs = a.partial_row_ptrs;
  c->x_scale = a.a_scale_ptr;
}
}  // namespace fmoe_detail

// Workspace bytes for one call; negative fmoe_status on error.
inline int64_t fused_moe_get_workspace_size(const fused_moe_traits& t, const fused_moe_args& a) {
  fmoe_traits_c tc; fmoe_args_c ac;
  int rc = fmoe_detail::to_c(t, &tc);
  if (rc != FMOE_OK) return rc;
  fmoe_detail::to_c(a, &ac);
  uint64_t bytes = 0;
  rc = fmoe_get_workspace_size(&tc, &ac, &bytes);
  return rc == FMOE_OK ? static_cast<int64_t>(bytes) : rc;
}

// The operator.  Returns elapsed ms (>= 0) when s.time_kernel, 0 when enqueued
// asynchronously, or a negative fmoe_status.
inline float fused_moe(const fused_moe_traits& t, const fused_moe_args& a, const stream_config& s) {
  fmoe_traits_c tc; fmoe_args_c ac;
  int rc = fmoe_detail::to_c(t, &tc);
  if (rc != FMOE_OK) return static_cast<float>(rc);
  fmoe_detail::to_c(a, &ac);
  float ms = 0.f;
  rc = fmoe_run(&tc, &ac, s.stream_id, s.time_kernel ? &ms : nullptr);
  return rc == FMOE_OK ? ms : static_cast<float>(rc);
}

struct moe_sorting_args {
  const int32_t* p_topk_ids = nullptr;       // [T, K]
  const float* p_weights = nullptr;          // [T, K]
  int32_t* p_sorted_token_ids = nullptr;     // [capacity]
  float* p_sorted_weights = nullptr;         // [capacity]
  int32_t* p_sorted_expert_ids = nullptr;    // [capacity / unit_size]
  int32_t* p_total_tokens_post_pad = nullptr;  // [1]
  int tokens = 0;
  int unit_size = 128;   // block_m
  int num_experts = 0;
  int topk = 0;
};

inline float moe_sorting(const moe_sorting_args& a, const stream_config& s) {
  int rc = fmoe_sort(a.p_topk_ids, a.p_weights, a.tokens, a.topk, a.num_experts, a.unit_size,
                     a.p_sorted_token_ids, a.p_sorted_weights, a.p_sorted_expert_ids,
                     a.p_total_tokens_post_pad, s.stream_id);
  return static_cast<float>(rc);
}
