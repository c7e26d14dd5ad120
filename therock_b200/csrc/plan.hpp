// Host-only part of the C-ABI: argument validation, workspace planning and the choice of
// kernel flavour.  Nothing here touches CUDA, so the same code is compiled into the library
// and into a plain g++ program that runs it under the address / undefined-behaviour
// sanitizers (tests/cpp/plan_sanitize.cpp).
#pragma once

#include <stdarg.h>
#include <stdint.h>
#include <stdio.h>

#include "../../include/fused_moe_c.h"

namespace fmoe {

constexpr int kPlanBlockM = 128;     // rows per sorted block == M of one MMA tile
constexpr int kPlanSlabRows = 128;   // rows of one weight slab
constexpr int kPlanTileN = 256;      // accumulator columns of one tile
constexpr int kSortMultiCtaPairs = 8192;   // pairs from which moe_sorting spreads over several CTAs
constexpr int kSortMaxCtasPlan = 64;
constexpr bool kFusedBlockQuant = true;    // 1x128 quantisation of the intermediate inside gemm1's epilogue

// Text of the last error on this thread (shared by every translation unit of the library).
inline char* last_error_buf() {
  static thread_local char buf[512] = "";
  return buf;
}
inline int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(last_error_buf(), 512, fmt, ap);
  va_end(ap);
  return code;
}

inline uint64_t align256(uint64_t v) { return (v + 255) & ~static_cast<uint64_t>(255); }

inline bool quant_is_fp8(int q) { return q != FMOE_QUANT_NONE; }
inline bool quant_is_block(int q) { return q == FMOE_QUANT_BLOCK128 || q == FMOE_QUANT_BLOCK128_UE8M0; }

inline int64_t sort_capacity(int32_t T, int32_t K, int32_t E, int32_t block_m) {
  if (block_m <= 0) return 0;
  const int64_t c = static_cast<int64_t>(T) * K + static_cast<int64_t>(E) * (block_m - 1);
  return (c + block_m - 1) / block_m * block_m;
}

inline int validate_traits(const fmoe_traits_c* t) {
  if (!t) return fail(FMOE_ERR_INVALID_ARG, "traits is null");
  if (t->quant < FMOE_QUANT_NONE || t->quant > FMOE_QUANT_BLOCK128_UE8M0)
    return fail(FMOE_ERR_INVALID_ARG, "unknown quant mode %d", t->quant);
  const int want = t->quant == FMOE_QUANT_NONE ? FMOE_BF16 : FMOE_FP8_E4M3;
  if (t->weight_dtype != want)
    return fail(FMOE_ERR_INVALID_ARG, "weight_dtype %d does not match quant mode %d", t->weight_dtype, t->quant);
  if (t->activation != FMOE_ACT_SILU) return fail(FMOE_ERR_UNSUPPORTED, "only SiLU activation is built");
  if (t->gate_only != 0 && t->gate_only != 1) return fail(FMOE_ERR_INVALID_ARG, "gate_only must be 0 or 1");
  if (t->gate_only && quant_is_block(t->quant))
    return fail(FMOE_ERR_UNSUPPORTED, "gate_only with 128-wide block scales is not built");
  if (t->block_m != kPlanBlockM) return fail(FMOE_ERR_UNSUPPORTED, "block_m must be %d", kPlanBlockM);
  if (t->gemm_mode < 0 || t->gemm_mode > 2) return fail(FMOE_ERR_INVALID_ARG, "gemm_mode must be 0, 1 or 2");
  if (t->weight_layout != FMOE_WEIGHTS_ROW_MAJOR && t->weight_layout != FMOE_WEIGHTS_TILED128)
    return fail(FMOE_ERR_INVALID_ARG, "unknown weight layout %d", t->weight_layout);
  if (t->partial_dtype != FMOE_PARTIAL_F32 && t->partial_dtype != FMOE_PARTIAL_BF16)
    return fail(FMOE_ERR_INVALID_ARG, "unknown partial_dtype %d", t->partial_dtype);
  return FMOE_OK;
}

// K may exceed E: on the receiving side of a de-duplicated expert-parallel dispatch a row
// carries the token's K-wide id list with -1 where the expert lives elsewhere, and a rank may
// own fewer than K experts.  Ids outside [0, E) are skipped by every kernel.
inline int validate_dims(const fmoe_traits_c* t, const fmoe_args_c* a) {
  if (!a) return fail(FMOE_ERR_INVALID_ARG, "args is null");
  if (a->T < 0 || a->H <= 0 || a->I <= 0 || a->E <= 0 || a->K <= 0)
    return fail(FMOE_ERR_INVALID_ARG, "dimensions must be positive (T=%d H=%d I=%d E=%d K=%d)", a->T, a->H, a->I,
                a->E, a->K);
  if (a->E > 1024) return fail(FMOE_ERR_UNSUPPORTED, "at most 1024 experts");
  if (a->K > 1024) return fail(FMOE_ERR_UNSUPPORTED, "at most 1024 experts per token");
  if (a->I % kPlanSlabRows)
    return fail(FMOE_ERR_UNSUPPORTED, "intermediate size must be a multiple of %d", kPlanSlabRows);
  if (t->gate_only && a->I % kPlanTileN)
    return fail(FMOE_ERR_UNSUPPORTED, "gate_only needs an intermediate size that is a multiple of %d", kPlanTileN);
  if (a->H % kPlanTileN) return fail(FMOE_ERR_UNSUPPORTED, "hidden size must be a multiple of %d", kPlanTileN);
  if (static_cast<int64_t>(a->T) * a->K > (1 << 24)) return fail(FMOE_ERR_UNSUPPORTED, "T*K too large");
  if (t->weight_layout == FMOE_WEIGHTS_TILED128) {
    const int es = t->quant == FMOE_QUANT_NONE ? 2 : 1;
    if ((a->H * es) % 128 || (a->I * es) % 128)
      return fail(FMOE_ERR_UNSUPPORTED, "tiled weights need K extents that are multiples of 128 bytes");
  }
  if (quant_is_block(t->quant) && (a->H % 128 || a->I % 128))
    return fail(FMOE_ERR_UNSUPPORTED, "block scales need hidden and intermediate sizes that are multiples of 128");
  if (a->x_scale && (!quant_is_fp8(t->quant) || a->H % 16))
    return fail(FMOE_ERR_INVALID_ARG, "x_scale (pre-quantised activations) needs an fp8 quant mode and H a multiple of 16");
  return FMOE_OK;
}

struct Plan {
  int64_t cap = 0;
  fmoe_ws_layout_c l{};
};

// Bytes of the UE8M0 scale array of a [cap, k_elems] activation matrix: one byte per row and
// 128-wide K group, row-major, each row padded to a multiple of four bytes so that the scales of
// four consecutive K groups are one aligned 32-bit word.
inline int packed_scale_pitch(int k_elems) { return ((k_elems / 128) + 3) & ~3; }
inline uint64_t packed_scale_bytes(int64_t cap, int k_elems) {
  return static_cast<uint64_t>(cap) * static_cast<uint64_t>(packed_scale_pitch(k_elems));
}

// Decode-sized batches without block scales run sorting + gather (+ quantisation) as one kernel.
inline bool fused_prologue(const fmoe_traits_c* t, const fmoe_args_c* a) {
  return static_cast<long long>(a->T) * a->K <= 128 && a->x_scale == nullptr &&
         (t->quant == FMOE_QUANT_NONE || t->quant == FMOE_QUANT_TOKEN_CHANNEL);
}
// fp8, K >= 2 and not decode-sized: quantise the T token rows once, then gather e4m3 rows.
inline bool quantise_once(const fmoe_traits_c* t, const fmoe_args_c* a) {
  return quant_is_fp8(t->quant) && a->K >= 2 && !fused_prologue(t, a) && a->H % 16 == 0 && a->x_scale == nullptr;
}

inline int make_plan(const fmoe_traits_c* t, const fmoe_args_c* a, Plan* p) {
  const int64_t cap = sort_capacity(a->T, a->K, a->E, t->block_m);
  const bool fp8 = quant_is_fp8(t->quant);
  const bool blk = quant_is_block(t->quant);
  const bool hw = t->quant == FMOE_QUANT_BLOCK128_UE8M0;
  p->cap = cap;
  uint64_t off = 0;
  auto take = [&off](uint64_t bytes) { uint64_t o = off; off = align256(off + bytes); return o; };
  fmoe_ws_layout_c& l = p->l;
  l.capacity = cap;
  l.meta = take(64 * sizeof(int32_t));
  l.sorted_token_ids = take(cap * 4);
  l.sorted_weights = take(cap * 4);
  l.sorted_rows = take(cap * 4);
  l.sorted_expert_ids = take(cap / t->block_m * 4);
  l.mblk_cum = take((static_cast<uint64_t>(a->E) + 1) * 4);
  l.a_sorted = take(static_cast<uint64_t>(cap) * a->H * (fp8 ? 1 : 2));
  if (!fp8) l.a_scale = take(0);
  else if (hw) l.a_scale = take(packed_scale_bytes(cap, a->H));
  else l.a_scale = take(static_cast<uint64_t>(cap) * 4 * (blk ? a->H / 128 : 1));
  // block-scaled modes quantise the intermediate inside the first GEMM's epilogue: no bf16 copy
  l.y = take(blk && kFusedBlockQuant ? 0 : static_cast<uint64_t>(cap) * a->I * 2);
  l.y_quant = take(fp8 ? static_cast<uint64_t>(cap) * a->I : 0);
  if (!fp8) l.y_scale = take(0);
  else if (hw) l.y_scale = take(packed_scale_bytes(cap, a->I));
  else l.y_scale = take(static_cast<uint64_t>(cap) * 4 * (blk ? a->I / 128 : 1));
  l.slots = take(static_cast<uint64_t>(a->T) * a->K * a->H * (t->partial_dtype == FMOE_PARTIAL_BF16 ? 2 : 4));
  l.sort_scratch = take(static_cast<uint64_t>(2 * kSortMaxCtasPlan) * a->E * 4);
  // fp8 with several experts per token: the token rows are quantised once, then gathered as e4m3
  const bool once = quantise_once(t, a);
  l.x_quant = take(once ? static_cast<uint64_t>(a->T) * a->H : 0);
  if (!once) l.x_quant_scale = take(0);
  else if (hw) l.x_quant_scale = take(packed_scale_bytes(a->T, a->H));
  else l.x_quant_scale = take(static_cast<uint64_t>(a->T) * 4 * (blk ? a->H / 128 : 1));
  l.total_bytes = off;
  return FMOE_OK;
}

// Kernel flavour per GEMM.  The CTA-pair kernel moves a third less of the operands per flop
// (about 5 % faster per tile) but pads every expert to an even number of row blocks and has
// half as many schedulable units, so whether it wins is a question of wave counts: estimate the
// persistent waves of both flavours from the expected number of routed rows.
inline int pick_gemm_flavour(const fmoe_traits_c* t, const fmoe_args_c* a, int n_blocks, int sms, int forced) {
  if (t->quant == FMOE_QUANT_BLOCK128) return FMOE_KERNEL_BLOCK_PROMOTE;
  const long long rows = static_cast<long long>(a->T) * a->K;
  if (t->quant == FMOE_QUANT_BLOCK128_UE8M0) {
    // Tokens on N (gemm_mode 2) multiplies only live rows, rounded up to 16 per expert, where
    // tokens on M pads every expert to 128-row blocks.  It is never chosen automatically: with two
    // N <= 224 MMAs per K step that both re-read the token tile, its operand reads from shared
    // memory per multiply-add are a third higher at 128 tokens per chunk, which on the
    // DeepSeek-V3 shape (256 rows per expert) cancels the quarter of the rows it saves (first GEMM
    // 2.20 ms against 2.24 ms), and its second GEMM does not overlap the epilogue (2.42 against 1.54 ms).
    return forced == 2 ? FMOE_KERNEL_BLOCK_HW_TOKENS_N : FMOE_KERNEL_BLOCK_HW_SCALE;
  }
  if (forced == 2) return FMOE_KERNEL_PAIR;
  const bool decode = rows <= 32;
  if (forced == 1) return decode ? FMOE_KERNEL_SINGLE_DECODE : FMOE_KERNEL_SINGLE;
  const long long exp_rows = static_cast<long long>(a->expected_tokens > 0 ? a->expected_tokens : a->T) * a->K;
  // expected row blocks: full blocks plus half a block of padding per expert that is hit
  const long long hit = exp_rows < a->E ? exp_rows : a->E;
  long long m_blocks = (exp_rows + 64 * hit + 127) / 128;
  if (m_blocks < hit) m_blocks = hit;
  const long long pairs = (m_blocks + hit / 2 + 1) / 2;          // odd experts waste half a pair
  const long long waves_single = (m_blocks * n_blocks + sms - 1) / sms;
  const long long waves_pair = (pairs * n_blocks + sms / 2 - 1) / (sms / 2);
  if (waves_pair * 95 < waves_single * 100) return FMOE_KERNEL_PAIR;
  return decode ? FMOE_KERNEL_SINGLE_DECODE : FMOE_KERNEL_SINGLE;
}

inline int describe_run(const fmoe_traits_c* t, const fmoe_args_c* a, int sms, int forced, fmoe_run_info_c* info) {
  const int nb1 = t->gate_only ? a->I / kPlanTileN : a->I / kPlanSlabRows;
  info->gemm1_kernel = pick_gemm_flavour(t, a, nb1, sms, forced);
  info->gemm2_kernel = pick_gemm_flavour(t, a, a->H / kPlanTileN, sms, forced);
  const bool multi_sort = static_cast<long long>(a->T) * a->K >= kSortMultiCtaPairs;
  info->sort_launches = multi_sort ? 3 : 1;
  info->quant_y_launch = (t->quant == FMOE_QUANT_TOKEN_CHANNEL || (quant_is_block(t->quant) && !kFusedBlockQuant)) ? 1 : 0;
  // sort, gather(+quant), gemm1, [quant of the intermediate], gemm2, combine; decode-sized
  // batches without block scales run sort and gather as one kernel
  if (fused_prologue(t, a)) info->sort_launches = 0;
  info->launches = info->sort_launches + 1 + 1 + info->quant_y_launch + 1 + 1;
  if (quantise_once(t, a)) info->launches += 1;      // quantise the token rows, then gather them
  if (a->partial_row_ptrs) info->launches -= 1;      // scattered partial rows: no combine
  return FMOE_OK;
}

}  // namespace fmoe
