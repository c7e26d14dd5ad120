/*
 * CPU oracle for the fused-MoE hot path.  TEST INFRASTRUCTURE ONLY: nothing in the
 * shipped library links, loads or calls this file.  Only the tests, the smoke check and
 * the benchmark's CPU-baseline / reference arm use it, and only as the checker or as the
 * timed CPU baseline.
 *
 * PARITY UNPINNED.  The operator being restated is Composable Kernel's ck_tile fused-MoE
 * (moe_sorting + gate/up GEMM + SiLU*up + down GEMM + top-k weighted combine).  TheRock
 * only declares a build of that library (math-libs/CMakeLists.txt:553-620, source taken
 * from the rocm-libraries submodule, .gitmodules:19-22), and the submodule directory is
 * empty in the reference checkout, pinned commit unknown.  There is therefore no
 * reference source, golden vector or known-answer test to pin this file against.  Every
 * function below states the arithmetic contract it implements; the contract is this
 * repository's own and is cross-checked by an independent numpy restatement
 * (oracle/oracle.py) and by committed golden fixtures generated from it.
 *
 * Arithmetic contract
 *   bf16      : IEEE round-to-nearest-even from f32, NaN preserved.
 *   e4m3 (fn) : 1-4-3, bias 7, max 448, no inf; f32 -> e4m3 rounds to nearest even and
 *               saturates to +-448.
 *   routing   : softmax or sigmoid in f32, top-K by value, ties to the lower expert
 *               index, weights renormalised to sum 1.
 *   sorting   : stable counting sort of the T*K (token,k) pairs by expert id; each
 *               expert's bucket padded to a multiple of block_m; pad slots carry token
 *               id T and weight 0; ids outside [0,E) are dropped.
 *   bf16 path : gate/up = x . W1^T accumulated in f32; y = silu(gate)*up in f32, rounded
 *               to bf16; o = y . W2^T in f32; out = bf16( sum_k w_k * o_k ), k ascending.
 *   quantise  : s = absmax/448 (1 if all zero), r = 1/s in f32, q = e4m3(v * r).
 *               Power-of-two variant (mode 3, the MX "UE8M0" scale format): s is the smallest
 *               power of two >= absmax/448, exponent clamped to [-126, 127].
 *   fp8 paths : operands quantised (activations dynamically, weights given quantised),
 *               integer-exact products accumulated in f32, scales applied after the
 *               accumulation (per token x per channel) or per 128-deep K block
 *               (1x128 activation groups x 128x128 weight blocks).  The intermediate y is
 *               rounded to bf16 (as in the bf16 path) and then quantised dynamically.
 *   combine   : default: out = bf16( sum_k f32(w_k * o_k) ).  bf16-partial variant (what the
 *               expert-parallel path and the partial_dtype = bf16 trait compute): every
 *               w_k * o_k is rounded to bf16 first, the sum of those is f32, rounded once more.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define ORC_API __attribute__((visibility("default")))

/* ------------------------------------------------------------------ number formats */

static inline float bf16_to_f32(uint16_t h) {
  uint32_t u = ((uint32_t)h) << 16;
  float f;
  memcpy(&f, &u, 4);
  return f;
}

static inline uint16_t f32_to_bf16(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x0040u); /* NaN */
  uint32_t lsb = (u >> 16) & 1u;
  u += 0x7fffu + lsb;
  return (uint16_t)(u >> 16);
}

static float g_e4m3_lut[256];
static int g_lut_ready = 0;

static void build_lut(void) {
  if (g_lut_ready) return;
  for (int b = 0; b < 256; ++b) {
    int s = b >> 7, e = (b >> 3) & 15, m = b & 7;
    float v;
    if (e == 15 && m == 7) v = NAN;
    else if (e == 0) v = ldexpf((float)m, -9);           /* subnormal: m * 2^-9 */
    else v = ldexpf(1.0f + (float)m / 8.0f, e - 7);
    g_e4m3_lut[b] = s ? -v : v;
  }
  g_lut_ready = 1;
}

/* f32 -> e4m3fn, round to nearest even, saturate to +-448 (NaN -> 0x7f). */
static inline uint8_t f32_to_e4m3(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  uint8_t sign = (uint8_t)((u >> 24) & 0x80u);
  uint32_t a = u & 0x7fffffffu;
  if (a > 0x7f800000u) return (uint8_t)(sign | 0x7f);
  float af;
  memcpy(&af, &a, 4);
  if (af >= 448.0f) return (uint8_t)(sign | 0x7e);       /* saturate (also inf) */
  if (af < 0.015625f) {                                   /* below 2^-6: subnormal grid 2^-9 */
    float q = af * 512.0f;                                /* exact scaling */
    float r = nearbyintf(q);                              /* RNE under default rounding mode */
    int m = (int)r;                                       /* 0..8 ; 8 == smallest normal */
    return (uint8_t)(sign | (uint8_t)m);
  }
  int e;
  float fr = frexpf(af, &e);                              /* af = fr * 2^e, fr in [0.5,1) */
  float mant = fr * 16.0f;                                /* [8,16) */
  float r = nearbyintf(mant);                             /* RNE */
  int mi = (int)r;
  int ex = e - 1;                                         /* unbiased exponent */
  if (mi == 16) { mi = 8; ex += 1; }
  int be = ex + 7;
  if (be > 15 || (be == 15 && (mi - 8) > 6)) return (uint8_t)(sign | 0x7e);
  return (uint8_t)(sign | (uint8_t)(be << 3) | (uint8_t)(mi - 8));
}

ORC_API void orc_f32_to_bf16(const float* in, uint16_t* out, int64_t n) {
  for (int64_t i = 0; i < n; ++i) out[i] = f32_to_bf16(in[i]);
}
ORC_API void orc_bf16_to_f32(const uint16_t* in, float* out, int64_t n) {
  for (int64_t i = 0; i < n; ++i) out[i] = bf16_to_f32(in[i]);
}
ORC_API void orc_f32_to_e4m3(const float* in, uint8_t* out, int64_t n) {
  for (int64_t i = 0; i < n; ++i) out[i] = f32_to_e4m3(in[i]);
}
ORC_API void orc_e4m3_to_f32(const uint8_t* in, float* out, int64_t n) {
  build_lut();
  for (int64_t i = 0; i < n; ++i) out[i] = g_e4m3_lut[in[i]];
}

/* Quantise rows of an f32 matrix to e4m3 with one scale per `group` consecutive columns:
 * scale = absmax/448 (1.0 when the group is all zero), q = e4m3(v * (1/scale)), the
 * reciprocal rounded once to f32.
 * group == cols gives the per-token (or per-output-channel) mode, group == 128 the 1x128
 * mode.  scales has rows * (cols/group) entries. */
/* scale of one quantisation group from its absolute maximum; pow2: rounded up to a power of two */
static inline float scale_from_amax(float amax, int pow2) {
  if (!(amax > 0.0f)) return 1.0f;
  float t = amax / 448.0f;
  if (!pow2) return t;
  uint32_t u;
  memcpy(&u, &t, 4);
  uint32_t e = (u >> 23) + ((u & 0x7fffffu) ? 1u : 0u);
  if (e < 1u) e = 1u;
  if (e > 254u) e = 254u;
  u = e << 23;
  memcpy(&t, &u, 4);
  return t;
}

ORC_API void orc_quant_rows_e4m3_ex(const float* in, int64_t rows, int64_t cols, int64_t group, int pow2,
                                    uint8_t* q, float* scales);

ORC_API void orc_quant_rows_e4m3(const float* in, int64_t rows, int64_t cols, int64_t group,
                                 uint8_t* q, float* scales) {
  orc_quant_rows_e4m3_ex(in, rows, cols, group, 0, q, scales);
}

/* pow2 = 1: power-of-two scales (mode 3) */
ORC_API void orc_quant_rows_e4m3_ex(const float* in, int64_t rows, int64_t cols, int64_t group, int pow2,
                                    uint8_t* q, float* scales) {
  int64_t ng = cols / group;
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < rows; ++r) {
    for (int64_t g = 0; g < ng; ++g) {
      const float* p = in + r * cols + g * group;
      float amax = 0.0f;
      for (int64_t c = 0; c < group; ++c) {
        float a = fabsf(p[c]);
        if (a > amax) amax = a;
      }
      float s = scale_from_amax(amax, pow2);
      float inv = 1.0f / s;
      scales[r * ng + g] = s;
      uint8_t* o = q + r * cols + g * group;
      for (int64_t c = 0; c < group; ++c) o[c] = f32_to_e4m3(p[c] * inv);
    }
  }
}

/* Quantise a weight tensor [rows, cols] with one scale per 128x128 block. */
ORC_API void orc_quant_blocks_e4m3_ex(const float* in, int64_t rows, int64_t cols, int pow2,
                                      uint8_t* q, float* scales);
ORC_API void orc_quant_blocks_e4m3(const float* in, int64_t rows, int64_t cols,
                                   uint8_t* q, float* scales) {
  orc_quant_blocks_e4m3_ex(in, rows, cols, 0, q, scales);
}
ORC_API void orc_quant_blocks_e4m3_ex(const float* in, int64_t rows, int64_t cols, int pow2,
                                      uint8_t* q, float* scales) {
  int64_t rb = rows / 128, cb = cols / 128;
#pragma omp parallel for schedule(static)
  for (int64_t b = 0; b < rb * cb; ++b) {
    int64_t br = b / cb, bc = b % cb;
    float amax = 0.0f;
    for (int64_t r = 0; r < 128; ++r)
      for (int64_t c = 0; c < 128; ++c) {
        float a = fabsf(in[(br * 128 + r) * cols + bc * 128 + c]);
        if (a > amax) amax = a;
      }
    float s = scale_from_amax(amax, pow2);
    float inv = 1.0f / s;
    scales[b] = s;
    for (int64_t r = 0; r < 128; ++r)
      for (int64_t c = 0; c < 128; ++c) {
        int64_t i = (br * 128 + r) * cols + bc * 128 + c;
        q[i] = f32_to_e4m3(in[i] * inv);
      }
  }
}

/* ------------------------------------------------------------------ routing */

/* logits [T,E] f32 -> topk_ids [T,K] i32, topk_weight [T,K] f32.
 * mode 0: softmax over E; mode 1: sigmoid.  Top-K by score descending, ties to the lower
 * index; weights divided by their sum. */
ORC_API int orc_route(const float* logits, int T, int E, int K, int mode,
                      int32_t* ids, float* w) {
  if (K > E || K <= 0) return -1;
#pragma omp parallel for schedule(static)
  for (int t = 0; t < T; ++t) {
    const float* l = logits + (int64_t)t * E;
    float* s = (float*)malloc(sizeof(float) * (size_t)E);
    if (mode == 0) {
      float mx = l[0];
      for (int e = 1; e < E; ++e) if (l[e] > mx) mx = l[e];
      float sum = 0.0f;
      for (int e = 0; e < E; ++e) { s[e] = expf(l[e] - mx); sum += s[e]; }
      for (int e = 0; e < E; ++e) s[e] = s[e] / sum;
    } else {
      for (int e = 0; e < E; ++e) s[e] = 1.0f / (1.0f + expf(-l[e]));
    }
    float tot = 0.0f;
    for (int k = 0; k < K; ++k) {
      int best = -1;
      for (int e = 0; e < E; ++e) {
        int taken = 0;
        for (int j = 0; j < k; ++j) if (ids[(int64_t)t * K + j] == e) taken = 1;
        if (taken) continue;
        if (best < 0 || s[e] > s[best]) best = e;
      }
      ids[(int64_t)t * K + k] = best;
      w[(int64_t)t * K + k] = s[best];
      tot += s[best];
    }
    for (int k = 0; k < K; ++k) w[(int64_t)t * K + k] = w[(int64_t)t * K + k] / tot;
    free(s);
  }
  return 0;
}

/* ------------------------------------------------------------------ moe_sorting */

/* Capacity of the sorted arrays: every expert may waste block_m-1 pad slots. */
ORC_API int64_t orc_sort_capacity(int64_t T, int64_t K, int64_t E, int64_t block_m) {
  int64_t c = T * K + E * (block_m - 1);
  return (c + block_m - 1) / block_m * block_m;
}

/* Stable bucket of the R = T*K routed pairs by expert.
 * out: sorted_token_ids[cap] (pad/tail = T), sorted_weights[cap] (pad/tail = 0),
 *      sorted_rows[cap] (flat pair index t*K+k, pad/tail = -1),
 *      sorted_expert_ids[cap/block_m] (tail = -1), num_post_pad[0] = padded total,
 *      mblk_cum[E+1] = cumulative block count per expert.
 * Any output pointer except sorted_token_ids may be NULL. */
ORC_API int orc_moe_sorting(const int32_t* topk_ids, const float* topk_w, int T, int K, int E,
                            int block_m, int32_t* sorted_token_ids, float* sorted_weights,
                            int32_t* sorted_rows, int32_t* sorted_expert_ids,
                            int32_t* num_post_pad, int32_t* mblk_cum) {
  int64_t R = (int64_t)T * K;
  int64_t cap = orc_sort_capacity(T, K, E, block_m);
  int64_t* cnt = (int64_t*)calloc((size_t)E + 1, sizeof(int64_t));
  int64_t* off = (int64_t*)calloc((size_t)E + 1, sizeof(int64_t));
  for (int64_t r = 0; r < R; ++r) {
    int e = topk_ids[r];
    if (e >= 0 && e < E) cnt[e]++;
  }
  int64_t run = 0;
  if (mblk_cum) mblk_cum[0] = 0;
  for (int e = 0; e < E; ++e) {
    off[e] = run;
    int64_t blocks = (cnt[e] + block_m - 1) / block_m;
    for (int64_t b = 0; b < blocks; ++b)
      if (sorted_expert_ids) sorted_expert_ids[run / block_m + b] = e;
    run += blocks * block_m;
    if (mblk_cum) mblk_cum[e + 1] = (int32_t)(run / block_m);
  }
  if (num_post_pad) num_post_pad[0] = (int32_t)run;
  for (int64_t b = run / block_m; b < cap / block_m; ++b)
    if (sorted_expert_ids) sorted_expert_ids[b] = -1;
  for (int64_t p = 0; p < cap; ++p) {
    sorted_token_ids[p] = T;
    if (sorted_weights) sorted_weights[p] = 0.0f;
    if (sorted_rows) sorted_rows[p] = -1;
  }
  for (int64_t r = 0; r < R; ++r) {
    int e = topk_ids[r];
    if (e < 0 || e >= E) continue;
    int64_t p = off[e]++;
    sorted_token_ids[p] = (int32_t)(r / K);
    if (sorted_weights) sorted_weights[p] = topk_w[r];
    if (sorted_rows) sorted_rows[p] = (int32_t)r;
  }
  free(cnt);
  free(off);
  return 0;
}

/* ------------------------------------------------------------------ fused MoE */

/* dot of two f32 vectors with 16 fixed partial sums (vectorisable, deterministic). */
static inline float dot_f32(const float* a, const float* b, int64_t n) {
  float acc[16];
  for (int j = 0; j < 16; ++j) acc[j] = 0.0f;
  int64_t i = 0;
  for (; i + 16 <= n; i += 16)
    for (int j = 0; j < 16; ++j) acc[j] += a[i + j] * b[i + j];
  float s = 0.0f;
  for (int j = 0; j < 16; ++j) s += acc[j];
  for (; i < n; ++i) s += a[i] * b[i];
  return s;
}

static inline float silu_f32(float g) { return g / (1.0f + expf(-g)); }

enum { ORC_Q_NONE = 0, ORC_Q_TOKEN_CHANNEL = 1, ORC_Q_BLOCK128 = 2, ORC_Q_BLOCK128_POW2 = 3 };

/* One expert applied to one token.
 *   xin : the token's activation row, f32 values (bf16-exact for mode 0, the e4m3 values
 *         for the fp8 modes); xs: activation scale(s) for the fp8 modes.
 *   w1/w2 point at the expert's weights (bf16 or e4m3 bytes), s1/s2 at its scales.
 * o[H] receives the un-weighted down-projection in f32. */
static void expert_forward(int quant, int gate_only, int H, int I, const float* xin, const float* xs,
                           const void* w1, const void* w2, const float* s1, const float* s2,
                           float* wrow, float* y, float* yq, float* ys, float* o) {
  const int HB = H / 128, IB = I / 128;
  /* gemm1 + SiLU*up (gate_only: W1 has I rows and y = SiLU(gate)) */
  for (int n = 0; n < I; ++n) {
    float gu[2] = {0.0f, 1.0f};
    for (int half = 0; half < (gate_only ? 1 : 2); ++half) {
      int64_t row = (int64_t)half * I + n;
      if (quant == ORC_Q_NONE) {
        const uint16_t* wr = (const uint16_t*)w1 + row * H;
        for (int k = 0; k < H; ++k) wrow[k] = bf16_to_f32(wr[k]);
        gu[half] = dot_f32(xin, wrow, H);
      } else {
        const uint8_t* wr = (const uint8_t*)w1 + row * H;
        for (int k = 0; k < H; ++k) wrow[k] = g_e4m3_lut[wr[k]];
        if (quant == ORC_Q_TOKEN_CHANNEL) {
          gu[half] = dot_f32(xin, wrow, H) * xs[0] * s1[row];
        } else {
          float acc = 0.0f;
          for (int kb = 0; kb < HB; ++kb)
            acc += dot_f32(xin + kb * 128, wrow + kb * 128, 128) * xs[kb] *
                   s1[(row / 128) * HB + kb];
          gu[half] = acc;
        }
      }
    }
    y[n] = gate_only ? silu_f32(gu[0]) : silu_f32(gu[0]) * gu[1];
  }
  /* intermediate rounding point: y is held as bf16 in every mode */
  for (int n = 0; n < I; ++n) y[n] = bf16_to_f32(f32_to_bf16(y[n]));
  if (quant == ORC_Q_NONE) {
    for (int n = 0; n < I; ++n) yq[n] = y[n];
  } else {
    int group = (quant == ORC_Q_TOKEN_CHANNEL) ? I : 128;
    for (int g = 0; g < I / group; ++g) {
      float amax = 0.0f;
      for (int c = 0; c < group; ++c) {
        float a = fabsf(y[g * group + c]);
        if (a > amax) amax = a;
      }
      float s = scale_from_amax(amax, quant == ORC_Q_BLOCK128_POW2);
      float inv = 1.0f / s;
      ys[g] = s;
      for (int c = 0; c < group; ++c)
        yq[g * group + c] = g_e4m3_lut[f32_to_e4m3(y[g * group + c] * inv)];
    }
  }
  /* gemm2 */
  for (int h = 0; h < H; ++h) {
    if (quant == ORC_Q_NONE) {
      const uint16_t* wr = (const uint16_t*)w2 + (int64_t)h * I;
      for (int k = 0; k < I; ++k) wrow[k] = bf16_to_f32(wr[k]);
      o[h] = dot_f32(yq, wrow, I);
    } else {
      const uint8_t* wr = (const uint8_t*)w2 + (int64_t)h * I;
      for (int k = 0; k < I; ++k) wrow[k] = g_e4m3_lut[wr[k]];
      if (quant == ORC_Q_TOKEN_CHANNEL) {
        o[h] = dot_f32(yq, wrow, I) * ys[0] * s2[h];
      } else {
        float acc = 0.0f;
        for (int kb = 0; kb < IB; ++kb)
          acc += dot_f32(yq + kb * 128, wrow + kb * 128, 128) * ys[kb] *
                 s2[(h / 128) * IB + kb];
        o[h] = acc;
      }
    }
  }
}

/* Fused MoE for a list of tokens.
 *   quant 0: w1 [E,2I,H] / w2 [E,H,I] bf16.
 *   quant 1: w1/w2 e4m3 bytes, w1_scale [E,2I], w2_scale [E,H]; activations quantised per
 *            token here (x and the intermediate y).
 *   quant 2: w1/w2 e4m3 bytes, w1_scale [E,2I/128,H/128], w2_scale [E,H/128,I/128];
 *            activations quantised per 1x128 group here.
 *   quant 3: as 2 with power-of-two scales.
 *   x [T,H] bf16; topk_ids/topk_w [T,K]; sel = n_sel token indices to evaluate (NULL = all
 *   T tokens in order); out [n_sel or T, H] bf16.
 * Expert ids outside [0,E) contribute nothing. */
ORC_API int orc_fused_moe_ex2(int T, int H, int I, int E, int K, int quant, int gate_only, int partial_bf16,
                              const uint16_t* x, const void* w1, const void* w2,
                              const float* w1_scale, const float* w2_scale,
                              const int32_t* topk_ids, const float* topk_w,
                              const int32_t* sel, int n_sel, uint16_t* out, int n_threads);

ORC_API int orc_fused_moe_ex(int T, int H, int I, int E, int K, int quant, int gate_only,
                             const uint16_t* x, const void* w1, const void* w2,
                             const float* w1_scale, const float* w2_scale,
                             const int32_t* topk_ids, const float* topk_w,
                             const int32_t* sel, int n_sel, uint16_t* out, int n_threads) {
  return orc_fused_moe_ex2(T, H, I, E, K, quant, gate_only, 0, x, w1, w2, w1_scale, w2_scale, topk_ids, topk_w, sel,
                           n_sel, out, n_threads);
}

ORC_API int orc_fused_moe(int T, int H, int I, int E, int K, int quant,
                          const uint16_t* x, const void* w1, const void* w2,
                          const float* w1_scale, const float* w2_scale,
                          const int32_t* topk_ids, const float* topk_w,
                          const int32_t* sel, int n_sel, uint16_t* out, int n_threads) {
  return orc_fused_moe_ex(T, H, I, E, K, quant, 0, x, w1, w2, w1_scale, w2_scale, topk_ids, topk_w, sel, n_sel,
                          out, n_threads);
}

/* gate_only = 1: W1 is [E, I, H] (no up projection) and y = SiLU(x . W1^T); weight scales of
 * W1 then have I rows per expert ([E, I] or [E, I/128, H/128]).
 * quant 3: as quant 2 with power-of-two activation scales (the weight scales passed in are
 * expected to be powers of two as well; they are used as given).
 * partial_bf16 = 1: every weighted expert output w_k * o_k is rounded to bf16 before the sum. */
ORC_API int orc_fused_moe_ex2(int T, int H, int I, int E, int K, int quant, int gate_only, int partial_bf16,
                              const uint16_t* x, const void* w1, const void* w2,
                              const float* w1_scale, const float* w2_scale,
                              const int32_t* topk_ids, const float* topk_w,
                              const int32_t* sel, int n_sel, uint16_t* out, int n_threads) {
  build_lut();
  const int w1_rows = gate_only ? I : 2 * I;
  if (quant < 0 || quant > 3) return -1;
  if (quant >= ORC_Q_BLOCK128 && (H % 128 || I % 128)) return -2;
  int n = sel ? n_sel : T;
  int maxd = H > I ? H : I;
  size_t wbytes = quant == ORC_Q_NONE ? 2 : 1;
#ifdef _OPENMP
  if (n_threads > 0) omp_set_num_threads(n_threads);
#endif
#pragma omp parallel
  {
    float* xin = (float*)malloc(sizeof(float) * (size_t)H);
    float* xs = (float*)malloc(sizeof(float) * (size_t)(H / 128 + 1));
    float* wrow = (float*)malloc(sizeof(float) * (size_t)maxd);
    float* y = (float*)malloc(sizeof(float) * (size_t)I);
    float* yq = (float*)malloc(sizeof(float) * (size_t)I);
    float* ys = (float*)malloc(sizeof(float) * (size_t)(I / 128 + 1));
    float* o = (float*)malloc(sizeof(float) * (size_t)H);
    float* acc = (float*)malloc(sizeof(float) * (size_t)H);
    uint8_t* q8 = (uint8_t*)malloc((size_t)H);
#pragma omp for schedule(dynamic, 1)
    for (int i = 0; i < n; ++i) {
      int t = sel ? sel[i] : i;
      const uint16_t* xr = x + (int64_t)t * H;
      for (int k = 0; k < H; ++k) xin[k] = bf16_to_f32(xr[k]);
      if (quant != ORC_Q_NONE) {
        int64_t group = quant == ORC_Q_TOKEN_CHANNEL ? H : 128;
        orc_quant_rows_e4m3_ex(xin, 1, H, group, quant == ORC_Q_BLOCK128_POW2, q8, xs);
        for (int k = 0; k < H; ++k) xin[k] = g_e4m3_lut[q8[k]];
      }
      for (int h = 0; h < H; ++h) acc[h] = 0.0f;
      for (int k = 0; k < K; ++k) {
        int e = topk_ids[(int64_t)t * K + k];
        if (e < 0 || e >= E) continue;
        float wk = topk_w[(int64_t)t * K + k];
        const uint8_t* w1e = (const uint8_t*)w1 + (size_t)e * w1_rows * H * wbytes;
        const uint8_t* w2e = (const uint8_t*)w2 + (size_t)e * H * I * wbytes;
        const float* s1 = NULL;
        const float* s2 = NULL;
        if (quant == ORC_Q_TOKEN_CHANNEL) {
          s1 = w1_scale + (size_t)e * w1_rows;
          s2 = w2_scale + (size_t)e * H;
        } else if (quant >= ORC_Q_BLOCK128) {
          s1 = w1_scale + (size_t)e * (w1_rows / 128) * (H / 128);
          s2 = w2_scale + (size_t)e * (H / 128) * (I / 128);
        }
        expert_forward(quant, gate_only, H, I, xin, xs, w1e, w2e, s1, s2, wrow, y, yq, ys, o);
        if (partial_bf16)
          for (int h = 0; h < H; ++h) acc[h] += bf16_to_f32(f32_to_bf16(wk * o[h]));
        else
          for (int h = 0; h < H; ++h) acc[h] += wk * o[h];
      }
      for (int h = 0; h < H; ++h) out[(int64_t)i * H + h] = f32_to_bf16(acc[h]);
    }
    free(xin); free(xs); free(wrow); free(y); free(yq); free(ys); free(o); free(acc); free(q8);
  }
  return 0;
}

ORC_API int orc_max_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}
