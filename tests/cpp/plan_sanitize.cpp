// Host-only exercise of the C-ABI's validation, workspace planning and kernel choice
// (therock_b200/csrc/plan.hpp), built with -fsanitize=address,undefined by
// tests/test_sanitizers.py.  Exits 0 when every expectation holds; the sanitizers abort the
// program on any out-of-bounds access, overflow or misaligned use they see on the way.
#include <cstdio>
#include <cstring>

#include "../../therock_b200/csrc/plan.hpp"

static int failures = 0;
#define EXPECT(cond)                                                          \
  do {                                                                        \
    if (!(cond)) { std::printf("FAILED line %d: %s\n", __LINE__, #cond); ++failures; } \
  } while (0)

static fmoe_traits_c traits(int quant) {
  fmoe_traits_c t;
  std::memset(&t, 0, sizeof(t));
  t.quant = quant;
  t.weight_dtype = quant == FMOE_QUANT_NONE ? FMOE_BF16 : FMOE_FP8_E4M3;
  t.block_m = 128;
  return t;
}

static fmoe_args_c dims(int T, int H, int I, int E, int K) {
  fmoe_args_c a;
  std::memset(&a, 0, sizeof(a));
  a.T = T; a.H = H; a.I = I; a.E = E; a.K = K;
  return a;
}

int main() {
  using namespace fmoe;
  // null and malformed arguments
  EXPECT(validate_traits(nullptr) == FMOE_ERR_INVALID_ARG);
  EXPECT(std::strlen(last_error_buf()) > 0);
  fmoe_traits_c t = traits(FMOE_QUANT_NONE);
  EXPECT(validate_traits(&t) == FMOE_OK);
  EXPECT(validate_dims(&t, nullptr) == FMOE_ERR_INVALID_ARG);
  for (int q = -3; q <= 6; ++q) {
    fmoe_traits_c tq = traits(q);
    const int rc = validate_traits(&tq);
    EXPECT((q >= 0 && q <= 3) ? rc == FMOE_OK : rc == FMOE_ERR_INVALID_ARG);
  }
  t.block_m = 64; EXPECT(validate_traits(&t) == FMOE_ERR_UNSUPPORTED); t.block_m = 128;
  t.partial_dtype = 9; EXPECT(validate_traits(&t) == FMOE_ERR_INVALID_ARG); t.partial_dtype = 0;
  t.gemm_mode = 3; EXPECT(validate_traits(&t) == FMOE_ERR_INVALID_ARG); t.gemm_mode = 0;
  t.weight_layout = -1; EXPECT(validate_traits(&t) == FMOE_ERR_INVALID_ARG); t.weight_layout = 0;

  // dimension limits, including the extremes that could overflow 32-bit products
  fmoe_args_c a = dims(128, 512, 1024, 8, 2);
  EXPECT(validate_dims(&t, &a) == FMOE_OK);
  a = dims(-1, 512, 1024, 8, 2); EXPECT(validate_dims(&t, &a) == FMOE_ERR_INVALID_ARG);
  a = dims(128, 500, 1024, 8, 2); EXPECT(validate_dims(&t, &a) == FMOE_ERR_UNSUPPORTED);
  a = dims(128, 512, 1000, 8, 2); EXPECT(validate_dims(&t, &a) == FMOE_ERR_UNSUPPORTED);
  a = dims(128, 512, 1024, 1025, 2); EXPECT(validate_dims(&t, &a) == FMOE_ERR_UNSUPPORTED);
  a = dims(128, 512, 1024, 2, 9); EXPECT(validate_dims(&t, &a) == FMOE_OK);      // K > E is legal
  a = dims(0x7fffffff, 512, 1024, 8, 0x7fffffff); EXPECT(validate_dims(&t, &a) == FMOE_ERR_UNSUPPORTED);
  a = dims(1 << 23, 512, 1024, 8, 2); EXPECT(validate_dims(&t, &a) == FMOE_OK);  // T*K == 2^24, the limit
  a = dims((1 << 23) + 1, 512, 1024, 8, 2); EXPECT(validate_dims(&t, &a) == FMOE_ERR_UNSUPPORTED);

  // workspace plans: regions ascend, are 256-byte aligned, do not overlap, and fit the total
  const int shapes[][5] = {{128, 512, 1024, 8, 2}, {4096, 4096, 14336, 8, 2}, {8192, 4096, 14336, 8, 2},
                           {16, 4096, 14336, 8, 2}, {8192, 7168, 2048, 256, 8}, {0, 256, 128, 1, 1},
                           {1 << 23, 16128, 16128, 1024, 2}};
  for (const auto& s : shapes) {
    for (int q = 0; q <= 3; ++q) {
      for (int pd = 0; pd <= 1; ++pd) {
        fmoe_traits_c tq = traits(q);
        tq.partial_dtype = pd;
        fmoe_args_c aq = dims(s[0], s[1], s[2], s[3], s[4]);
        if (validate_dims(&tq, &aq) != FMOE_OK) continue;
        Plan p;
        EXPECT(make_plan(&tq, &aq, &p) == FMOE_OK);
        const fmoe_ws_layout_c& l = p.l;
        const uint64_t offs[] = {l.meta, l.sorted_token_ids, l.sorted_weights, l.sorted_rows, l.sorted_expert_ids,
                                 l.mblk_cum, l.a_sorted, l.a_scale, l.y, l.y_quant, l.y_scale, l.slots,
                                 l.sort_scratch, l.x_quant, l.x_quant_scale, l.total_bytes};
        for (size_t i = 0; i + 1 < sizeof(offs) / sizeof(offs[0]); ++i) {
          EXPECT(offs[i] % 256 == 0);
          EXPECT(offs[i] <= offs[i + 1]);
        }
        EXPECT(l.capacity % 128 == 0);
        EXPECT(l.capacity >= static_cast<int64_t>(s[0]) * s[4]);
        EXPECT(l.slots + static_cast<uint64_t>(s[0]) * s[4] * s[1] * (pd ? 2 : 4) <= l.sort_scratch);
        fmoe_run_info_c info;
        std::memset(&info, 0, sizeof(info));
        EXPECT(describe_run(&tq, &aq, 148, 0, &info) == FMOE_OK);
        EXPECT(info.gemm1_kernel >= FMOE_KERNEL_SINGLE && info.gemm1_kernel <= FMOE_KERNEL_BLOCK_HW_TOKENS_N);
        EXPECT(info.launches >= 4 && info.launches <= 9);   // decode prologue (one launch for sort + gather) up to multi-CTA sort + quantise-once + quantised intermediate
        if (q == FMOE_QUANT_BLOCK128_UE8M0) {
          EXPECT(info.gemm1_kernel == FMOE_KERNEL_BLOCK_HW_SCALE);
          fmoe_run_info_c forced;
          std::memset(&forced, 0, sizeof(forced));
          EXPECT(describe_run(&tq, &aq, 148, 1, &forced) == FMOE_OK && forced.gemm1_kernel == FMOE_KERNEL_BLOCK_HW_SCALE);
          EXPECT(describe_run(&tq, &aq, 148, 2, &forced) == FMOE_OK && forced.gemm2_kernel == FMOE_KERNEL_BLOCK_HW_TOKENS_N);
        }
      }
    }
  }
  // pre-quantised activations: fp8 modes only; no quantise-once pass, no decode prologue, no x_quant region
  {
    fmoe_traits_c tq = t;
    int dummy = 0;
    fmoe_args_c aq = dims(16, 512, 256, 8, 2);
    aq.x_scale = &dummy;
    tq.quant = FMOE_QUANT_NONE; tq.weight_dtype = FMOE_BF16;
    EXPECT(validate_dims(&tq, &aq) == FMOE_ERR_INVALID_ARG);
    tq.quant = FMOE_QUANT_TOKEN_CHANNEL; tq.weight_dtype = FMOE_FP8_E4M3;
    EXPECT(validate_dims(&tq, &aq) == FMOE_OK);
    EXPECT(!fused_prologue(&tq, &aq) && !quantise_once(&tq, &aq));
    Plan p;
    EXPECT(make_plan(&tq, &aq, &p) == FMOE_OK && p.l.x_quant_scale == p.l.x_quant);
    fmoe_run_info_c info;
    std::memset(&info, 0, sizeof(info));
    EXPECT(describe_run(&tq, &aq, 148, 0, &info) == FMOE_OK && info.launches == 6);   // sort, gather, gemm1, quant y, gemm2, combine
    aq.x_scale = nullptr;
    EXPECT(fused_prologue(&tq, &aq));
  }
  // UE8M0 scale rows are padded to whole 32-bit words
  EXPECT(packed_scale_pitch(7 * 128) == 8 && packed_scale_pitch(16 * 128) == 16 && packed_scale_pitch(128) == 4);
  EXPECT(packed_scale_bytes(256, 7 * 128) == 256u * 8u);
  std::printf(failures ? "%d expectation(s) failed\n" : "ok\n", failures);
  return failures ? 1 : 0;
}
