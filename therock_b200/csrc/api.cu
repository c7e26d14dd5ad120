// C-ABI of libfmoe_b200.so: argument validation, workspace planning and the launch
// sequence of the fused-MoE operator.  No device memory is allocated here; every buffer
// belongs to the caller.
#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <mutex>

#include "../../include/fused_moe_c.h"
#include "gemm.cuh"
#include "internal.h"

namespace {

thread_local char g_err[512] = "";

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}

inline uint64_t align256(uint64_t v) { return (v + 255) & ~static_cast<uint64_t>(255); }

struct Plan {
  int64_t cap = 0;
  fmoe_ws_layout_c l{};
};

int validate_traits(const fmoe_traits_c* t) {
  if (!t) return fail(FMOE_ERR_INVALID_ARG, "traits is null");
  if (t->quant < FMOE_QUANT_NONE || t->quant > FMOE_QUANT_BLOCK128)
    return fail(FMOE_ERR_INVALID_ARG, "unknown quant mode %d", t->quant);
  const int want = t->quant == FMOE_QUANT_NONE ? FMOE_BF16 : FMOE_FP8_E4M3;
  if (t->weight_dtype != want)
    return fail(FMOE_ERR_INVALID_ARG, "weight_dtype %d does not match quant mode %d", t->weight_dtype, t->quant);
  if (t->activation != FMOE_ACT_SILU) return fail(FMOE_ERR_UNSUPPORTED, "only SiLU activation is built");
  if (t->gate_only != 0 && t->gate_only != 1) return fail(FMOE_ERR_INVALID_ARG, "gate_only must be 0 or 1");
  if (t->gate_only && t->quant == FMOE_QUANT_BLOCK128)
    return fail(FMOE_ERR_UNSUPPORTED, "gate_only with block128 scales is not built");
  if (t->block_m != fmoe::kBlockM) return fail(FMOE_ERR_UNSUPPORTED, "block_m must be %d", fmoe::kBlockM);
  if (t->gemm_mode < 0 || t->gemm_mode > 2) return fail(FMOE_ERR_INVALID_ARG, "gemm_mode must be 0, 1 or 2");
  if (t->weight_layout != FMOE_WEIGHTS_ROW_MAJOR && t->weight_layout != FMOE_WEIGHTS_TILED128)
    return fail(FMOE_ERR_INVALID_ARG, "unknown weight layout %d", t->weight_layout);
  return FMOE_OK;
}

int validate_dims(const fmoe_traits_c* t, const fmoe_args_c* a) {
  if (!a) return fail(FMOE_ERR_INVALID_ARG, "args is null");
  if (a->T < 0 || a->H <= 0 || a->I <= 0 || a->E <= 0 || a->K <= 0)
    return fail(FMOE_ERR_INVALID_ARG, "dimensions must be positive (T=%d H=%d I=%d E=%d K=%d)", a->T, a->H, a->I, a->E, a->K);
  if (a->K > a->E) return fail(FMOE_ERR_INVALID_ARG, "topk %d exceeds experts %d", a->K, a->E);
  if (a->E > 1024) return fail(FMOE_ERR_UNSUPPORTED, "at most 1024 experts");
  if (a->I % fmoe::kSlabRows) return fail(FMOE_ERR_UNSUPPORTED, "intermediate size must be a multiple of %d", fmoe::kSlabRows);
  if (t->gate_only && a->I % fmoe::kTileN)
    return fail(FMOE_ERR_UNSUPPORTED, "gate_only needs an intermediate size that is a multiple of %d", fmoe::kTileN);
  if (a->H % fmoe::kTileN) return fail(FMOE_ERR_UNSUPPORTED, "hidden size must be a multiple of %d", fmoe::kTileN);
  if (static_cast<int64_t>(a->T) * a->K > (1 << 24)) return fail(FMOE_ERR_UNSUPPORTED, "T*K too large");
  if (t->weight_layout == FMOE_WEIGHTS_TILED128) {
    const int es = t->quant == FMOE_QUANT_NONE ? 2 : 1;
    if ((a->H * es) % 128 || (a->I * es) % 128)
      return fail(FMOE_ERR_UNSUPPORTED, "tiled weights need K extents that are multiples of 128 bytes");
  }
  if (t->quant == FMOE_QUANT_BLOCK128 && (a->H % 128 || a->I % 128))
    return fail(FMOE_ERR_UNSUPPORTED, "block128 needs hidden and intermediate sizes that are multiples of 128");
  return FMOE_OK;
}

int make_plan(const fmoe_traits_c* t, const fmoe_args_c* a, Plan* p) {
  const int64_t cap = fmoe_sort_capacity(a->T, a->K, a->E, t->block_m);
  const bool fp8 = t->quant != FMOE_QUANT_NONE;
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
  l.mblk_cum = take((a->E + 1) * 4);
  l.a_sorted = take(static_cast<uint64_t>(cap) * a->H * (fp8 ? 1 : 2));
  const bool blk = t->quant == FMOE_QUANT_BLOCK128;
  l.a_scale = take(fp8 ? static_cast<uint64_t>(cap) * 4 * (blk ? a->H / 128 : 1) : 0);
  l.y = take(static_cast<uint64_t>(cap) * a->I * 2);
  l.y_quant = take(fp8 ? static_cast<uint64_t>(cap) * a->I : 0);
  l.y_scale = take(fp8 ? static_cast<uint64_t>(cap) * 4 * (blk ? a->I / 128 : 1) : 0);
  l.slots = take(static_cast<uint64_t>(a->T) * a->K * a->H * 4);
  l.sort_scratch = take(fmoe::sort_scratch_words(a->E) * 4);
  l.total_bytes = off;
  return FMOE_OK;
}

int set_device_for(const void* ptr) {
  cudaPointerAttributes attr;
  if (cudaPointerGetAttributes(&attr, ptr) != cudaSuccess) {
    cudaGetLastError();
    return FMOE_OK;   // not fatal: keep the calling thread's device
  }
  if (attr.type == cudaMemoryTypeDevice) {
    int cur = -1;
    cudaGetDevice(&cur);
    if (cur != attr.device && cudaSetDevice(attr.device) != cudaSuccess)
      return fail(FMOE_ERR_CUDA, "cudaSetDevice(%d) failed", attr.device);
  }
  return FMOE_OK;
}

#define FMOE_CUDA(expr)                                                                    \
  do {                                                                                     \
    cudaError_t e__ = (expr);                                                              \
    if (e__ != cudaSuccess)                                                                \
      return fail(FMOE_ERR_CUDA, "%s failed: %s", #expr, cudaGetErrorString(e__));         \
  } while (0)

}  // namespace

extern "C" {

int fmoe_version(void) { return 100; }

const char* fmoe_last_error(void) { return g_err; }

int64_t fmoe_sort_capacity(int32_t T, int32_t K, int32_t E, int32_t block_m) {
  if (block_m <= 0) return 0;
  const int64_t c = static_cast<int64_t>(T) * K + static_cast<int64_t>(E) * (block_m - 1);
  return (c + block_m - 1) / block_m * block_m;
}

int fmoe_sort(const int32_t* topk_ids, const float* topk_weight, int32_t T, int32_t K, int32_t E,
              int32_t block_m, int32_t* sorted_token_ids, float* sorted_weights,
              int32_t* sorted_expert_ids, int32_t* num_tokens_post_pad, void* stream) {
  if (!topk_ids || !sorted_token_ids) return fail(FMOE_ERR_INVALID_ARG, "topk_ids and sorted_token_ids are required");
  if (sorted_weights && !topk_weight) return fail(FMOE_ERR_INVALID_ARG, "sorted_weights requested without topk_weight");
  if (T < 0 || K <= 0 || E <= 0 || block_m <= 0) return fail(FMOE_ERR_INVALID_ARG, "bad dimensions");
  if (E > 1024) return fail(FMOE_ERR_UNSUPPORTED, "at most 1024 experts");
  if (static_cast<int64_t>(T) * K > (1 << 24)) return fail(FMOE_ERR_UNSUPPORTED, "T*K too large");
  int rc = set_device_for(topk_ids);
  if (rc != FMOE_OK) return rc;
  FMOE_CUDA(fmoe::launch_moe_sorting(topk_ids, topk_weight, T, K, E, block_m,
                                     fmoe_sort_capacity(T, K, E, block_m), sorted_token_ids,
                                     sorted_weights, nullptr, sorted_expert_ids, num_tokens_post_pad,
                                     nullptr, nullptr, static_cast<cudaStream_t>(stream)));
  return FMOE_OK;
}

int fmoe_get_workspace_layout(const fmoe_traits_c* traits, const fmoe_args_c* args,
                              fmoe_ws_layout_c* layout) {
  int rc = validate_traits(traits);
  if (rc == FMOE_OK) rc = validate_dims(traits, args);
  if (rc != FMOE_OK) return rc;
  if (!layout) return fail(FMOE_ERR_INVALID_ARG, "layout is null");
  Plan p;
  make_plan(traits, args, &p);
  *layout = p.l;
  return FMOE_OK;
}

int fmoe_get_workspace_size(const fmoe_traits_c* traits, const fmoe_args_c* args, uint64_t* bytes) {
  if (!bytes) return fail(FMOE_ERR_INVALID_ARG, "bytes is null");
  fmoe_ws_layout_c l;
  int rc = fmoe_get_workspace_layout(traits, args, &l);
  if (rc != FMOE_OK) return rc;
  *bytes = l.total_bytes;
  return FMOE_OK;
}

int fmoe_launches_per_run(const fmoe_traits_c* traits) {
  if (validate_traits(traits) != FMOE_OK) return FMOE_ERR_INVALID_ARG;
  // sort, gather(+quant), gemm1, [quant of the intermediate], gemm2, combine
  return traits->quant == FMOE_QUANT_NONE ? 5 : 6;
}

// Stage boundaries at which run_impl records an event when given an event array:
// 0 start, 1 after sort, 2 after gather, 3 after gemm1, 4 after quant of y (== 3 for bf16),
// 5 after gemm2, 6 after combine.
constexpr int kStageEvents = 7;

static int run_impl(const fmoe_traits_c* traits, const fmoe_args_c* args, void* stream_v, float* ms_out,
                    cudaEvent_t* stage_ev) {
  int rc = validate_traits(traits);
  if (rc == FMOE_OK) rc = validate_dims(traits, args);
  if (rc != FMOE_OK) return rc;
  const fmoe_args_c& a = *args;
  if (a.T == 0) {   // nothing to do; an empty batch may legitimately come with null pointers
    if (stage_ev)
      for (int i = 0; i < kStageEvents; ++i) FMOE_CUDA(cudaEventRecord(stage_ev[i], static_cast<cudaStream_t>(stream_v)));
    if (ms_out) *ms_out = 0.f;
    return FMOE_OK;
  }
  if (!a.x || !a.w1 || !a.w2 || !a.topk_ids || !a.topk_weight || !a.out)
    return fail(FMOE_ERR_INVALID_ARG, "x, w1, w2, topk_ids, topk_weight and out are required");
  const bool fp8 = traits->quant != FMOE_QUANT_NONE;
  if (fp8 && (!a.w1_scale || !a.w2_scale)) return fail(FMOE_ERR_INVALID_ARG, "fp8 variants need w1_scale and w2_scale");
  Plan plan;
  make_plan(traits, args, &plan);
  if (!a.workspace) return fail(FMOE_ERR_WORKSPACE, "workspace is null (%llu bytes needed)", (unsigned long long)plan.l.total_bytes);
  if (a.workspace_bytes < plan.l.total_bytes)
    return fail(FMOE_ERR_WORKSPACE, "workspace has %llu bytes, %llu needed", (unsigned long long)a.workspace_bytes,
                (unsigned long long)plan.l.total_bytes);
  if (reinterpret_cast<uintptr_t>(a.workspace) & 255) return fail(FMOE_ERR_WORKSPACE, "workspace must be 256-byte aligned");

  rc = set_device_for(a.x);
  if (rc != FMOE_OK) return rc;

  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
  uint8_t* ws = static_cast<uint8_t*>(a.workspace);
  const fmoe_ws_layout_c& l = plan.l;
  int32_t* meta = reinterpret_cast<int32_t*>(ws + l.meta);
  int32_t* num_post_pad = meta + 0;
  int32_t* status = meta + 1;
  int32_t* sorted_ids = reinterpret_cast<int32_t*>(ws + l.sorted_token_ids);
  float* sorted_w = reinterpret_cast<float*>(ws + l.sorted_weights);
  int32_t* sorted_rows = reinterpret_cast<int32_t*>(ws + l.sorted_rows);
  int32_t* expert_ids = reinterpret_cast<int32_t*>(ws + l.sorted_expert_ids);
  int32_t* mblk_cum = reinterpret_cast<int32_t*>(ws + l.mblk_cum);
  void* a_sorted = ws + l.a_sorted;
  float* a_scale = fp8 ? reinterpret_cast<float*>(ws + l.a_scale) : nullptr;
  void* y = ws + l.y;
  void* yq = ws + l.y_quant;
  float* y_scale = fp8 ? reinterpret_cast<float*>(ws + l.y_scale) : nullptr;
  float* slots = reinterpret_cast<float*>(ws + l.slots);

#define FMOE_STAGE(i) do { if (stage_ev) FMOE_CUDA(cudaEventRecord(stage_ev[i], stream)); } while (0)
  cudaEvent_t ev0 = nullptr, ev1 = nullptr;
  FMOE_STAGE(0);
  if (ms_out) {
    FMOE_CUDA(cudaEventCreate(&ev0));
    FMOE_CUDA(cudaEventCreate(&ev1));
    FMOE_CUDA(cudaEventRecord(ev0, stream));
  }

  FMOE_CUDA(fmoe::launch_moe_sorting(a.topk_ids, a.topk_weight, a.T, a.K, a.E, traits->block_m, plan.cap,
                                     sorted_ids, sorted_w, sorted_rows, expert_ids, num_post_pad,
                                     mblk_cum, status, stream, a.num_tokens_dev, 1, nullptr,
                                     reinterpret_cast<int32_t*>(ws + l.sort_scratch)));
  FMOE_STAGE(1);
  const bool blk = traits->quant == FMOE_QUANT_BLOCK128;
  const int qmode = !fp8 ? 0 : (blk ? 2 : 1);
  FMOE_CUDA(fmoe::launch_gather_rows(a.x, a.T, a.H, sorted_ids, num_post_pad, plan.cap, qmode,
                                     a_sorted, a_scale, stream));
  FMOE_STAGE(2);

  fmoe::GemmLaunch g{};
  int drv = 0;
  g.fp8 = fp8;
  g.b_tiled = traits->weight_layout == FMOE_WEIGHTS_TILED128;
  g.block_scale = blk;
  g.num_experts = a.E;
  g.mblk_cum = mblk_cum;
  g.sorted_rows = sorted_rows;
  g.sorted_weights = sorted_w;
  g.status = status;
  g.max_m_blocks = static_cast<int>(plan.cap / fmoe::kBlockM);
  // no expert can receive more rows than there are routed pairs: lets decode-sized batches
  // stage only the rows that can be real
  g.max_live_rows = static_cast<long long>(a.T) * a.K <= fmoe::kBlockM ? a.T * a.K : 0;
  // Kernel flavour per GEMM.  The CTA-pair kernel moves a third less of the operands per flop
  // (about 5 % faster per tile) but pads every expert to an even number of row blocks and
  // has half as many schedulable units, so whether it wins is a question of wave counts:
  // estimate the persistent waves of both flavours from the expected number of routed rows.
  const int forced_mode = traits->gemm_mode ? traits->gemm_mode : fmoe::gemm_mode_from_env();
  const long long exp_rows = static_cast<long long>(a.expected_tokens > 0 ? a.expected_tokens : a.T) * a.K;
  const int sms = fmoe::device_sm_count();
  auto pick_mode = [&](int n_blocks) {
    if (forced_mode) return forced_mode;
    // expected row blocks: full blocks plus half a block of padding per expert that is hit
    const long long hit = exp_rows < a.E ? exp_rows : a.E;
    long long m_blocks = (exp_rows + 64 * hit + 127) / 128;
    if (m_blocks < hit) m_blocks = hit;                             // at least one block per expert hit
    const long long pairs = (m_blocks + hit / 2 + 1) / 2;          // odd experts waste half a pair
    const long long waves_single = (m_blocks * n_blocks + sms - 1) / sms;
    const long long waves_pair = (pairs * n_blocks + sms / 2 - 1) / (sms / 2);
    return (waves_pair * 95 < waves_single * 100) ? 2 : 1;
  };
  // gemm1: [cap, H] x W1[E, 2I, H]^T -> SiLU(gate) * up -> y [cap, I]
  if (traits->gate_only) {
    // W1 is [E, I, H]: a tile is 256 consecutive gate rows, y = SiLU(gate)
    g.mode = pick_mode(a.I / fmoe::kTileN);
    g.epilogue = fmoe::kEpiSilu;
    g.b_rows_per_expert = a.I;
    g.n_blocks = a.I / fmoe::kTileN; g.n_stride = fmoe::kTileN; g.second_slab_offset = fmoe::kSlabRows;
  } else {
    g.mode = pick_mode(a.I / fmoe::kSlabRows);
    g.epilogue = fmoe::kEpiSiluMul;
    g.b_rows_per_expert = 2 * a.I;
    g.n_blocks = a.I / fmoe::kSlabRows; g.n_stride = fmoe::kSlabRows; g.second_slab_offset = a.I;
  }
  g.a = a_sorted; g.a_rows = plan.cap; g.b = a.w1; g.k_elems = a.H;
  g.a_scale = a_scale; g.b_scale = fp8 ? a.w1_scale : nullptr;
  g.out = y; g.ld_out = a.I;
  if (fmoe::launch_grouped_gemm(g, stream, &drv) != cudaSuccess)
    return fail(FMOE_ERR_CUDA, "gemm1 launch failed (cuda: %s, driver code %d)", cudaGetErrorString(cudaGetLastError()), drv);
  FMOE_STAGE(3);

  const void* a2 = y;
  if (fp8) {
    FMOE_CUDA(fmoe::launch_gather_rows(y, static_cast<int>(plan.cap), a.I, nullptr, num_post_pad, plan.cap, qmode,
                                       yq, y_scale, stream, sorted_rows));
    a2 = yq;
  }
  FMOE_STAGE(4);
  // gemm2: [cap, I] x W2[E, H, I]^T * topk_weight -> slots [T*K, H]
  g.mode = pick_mode(a.H / fmoe::kTileN);
  g.epilogue = fmoe::kEpiScaledSlots;
  g.a = a2; g.b = a.w2; g.k_elems = a.I;
  g.b_rows_per_expert = a.H;
  g.n_blocks = a.H / fmoe::kTileN; g.n_stride = fmoe::kTileN; g.second_slab_offset = fmoe::kSlabRows;
  g.a_scale = y_scale; g.b_scale = fp8 ? a.w2_scale : nullptr;
  g.out = slots; g.ld_out = a.H;
  if (fmoe::launch_grouped_gemm(g, stream, &drv) != cudaSuccess)
    return fail(FMOE_ERR_CUDA, "gemm2 launch failed (cuda: %s, driver code %d)", cudaGetErrorString(cudaGetLastError()), drv);
  FMOE_STAGE(5);

  FMOE_CUDA(fmoe::launch_combine(slots, a.topk_ids, a.T, a.K, a.E, a.H, a.out, stream, a.num_tokens_dev));
  FMOE_STAGE(6);
#undef FMOE_STAGE

  if (ms_out) {
    FMOE_CUDA(cudaEventRecord(ev1, stream));
    FMOE_CUDA(cudaEventSynchronize(ev1));
    FMOE_CUDA(cudaEventElapsedTime(ms_out, ev0, ev1));
    cudaEventDestroy(ev0);
    cudaEventDestroy(ev1);
    int32_t st = 0;
    FMOE_CUDA(cudaMemcpy(&st, status, sizeof(st), cudaMemcpyDeviceToHost));
    if (st != 0) return fail(FMOE_ERR_DEVICE_TIMEOUT, "device status word 0x%x: a bounded wait ran out", st);
  }
  return FMOE_OK;
}

int fmoe_run(const fmoe_traits_c* traits, const fmoe_args_c* args, void* stream, float* ms_out) {
  return run_impl(traits, args, stream, ms_out, nullptr);
}

// ---- per-stage timing: events are recorded between the kernels of each run and read back
// later, so the timed loop itself never synchronises.
struct fmoe_profile {
  int max_runs;
  int runs;
  cudaEvent_t* ev;   // [max_runs][kStageEvents]
};

int fmoe_profile_create(int32_t max_runs, void** handle) {
  if (!handle || max_runs <= 0) return fail(FMOE_ERR_INVALID_ARG, "handle and a positive run count are required");
  fmoe_profile* p = new fmoe_profile{max_runs, 0, new cudaEvent_t[static_cast<size_t>(max_runs) * kStageEvents]};
  for (int i = 0; i < max_runs * kStageEvents; ++i) {
    if (cudaEventCreate(&p->ev[i]) != cudaSuccess) return fail(FMOE_ERR_CUDA, "cudaEventCreate failed");
  }
  *handle = p;
  return FMOE_OK;
}

int fmoe_run_profiled(const fmoe_traits_c* traits, const fmoe_args_c* args, void* stream, void* handle) {
  fmoe_profile* p = static_cast<fmoe_profile*>(handle);
  if (!p) return fail(FMOE_ERR_INVALID_ARG, "profile handle is null");
  if (p->runs >= p->max_runs) return fail(FMOE_ERR_INVALID_ARG, "profile handle is full (%d runs)", p->max_runs);
  int rc = run_impl(traits, args, stream, nullptr, p->ev + static_cast<size_t>(p->runs) * kStageEvents);
  if (rc == FMOE_OK) p->runs++;
  return rc;
}

int fmoe_profile_read(void* handle, float* stage_ms, int32_t* runs) {
  fmoe_profile* p = static_cast<fmoe_profile*>(handle);
  if (!p || !stage_ms) return fail(FMOE_ERR_INVALID_ARG, "handle and stage_ms are required");
  for (int sidx = 0; sidx < kStageEvents - 1; ++sidx) stage_ms[sidx] = 0.f;
  for (int r = 0; r < p->runs; ++r) {
    cudaEvent_t* e = p->ev + static_cast<size_t>(r) * kStageEvents;
    FMOE_CUDA(cudaEventSynchronize(e[kStageEvents - 1]));
    for (int sidx = 0; sidx < kStageEvents - 1; ++sidx) {
      float ms = 0.f;
      FMOE_CUDA(cudaEventElapsedTime(&ms, e[sidx], e[sidx + 1]));
      stage_ms[sidx] += ms;
    }
  }
  if (runs) *runs = p->runs;
  p->runs = 0;
  return FMOE_OK;
}

int fmoe_profile_destroy(void* handle) {
  fmoe_profile* p = static_cast<fmoe_profile*>(handle);
  if (!p) return FMOE_OK;
  for (int i = 0; i < p->max_runs * kStageEvents; ++i) cudaEventDestroy(p->ev[i]);
  delete[] p->ev;
  delete p;
  return FMOE_OK;
}

// ---- entry point that allocates nothing: the workspace lives inside the library image.
//
// Some hosts of this operator are not allowed to obtain device memory at all: a plugin
// slot in a serving engine that hands the operator only its input and output tensors, a
// foreign-function caller with no CUDA allocator of its own, or a latency-critical loop in
// which cudaMalloc is banned because it synchronises the whole device.  For them the
// scratch the operator needs is this fixed array.  It is part of the loaded module, so
// every GPU that loads the library keeps these FMOE_STATIC_WS_BYTES reserved until the
// process exits, which is why the limit is modest.
static __device__ __align__(256) unsigned char g_fmoe_static_ws[FMOE_STATIC_WS_BYTES];

namespace {
constexpr int kStaticWsMaxDevices = 64;
void* g_static_ws_addr[kStaticWsMaxDevices] = {nullptr};   // device address of the array, per GPU
std::mutex g_static_ws_mu;
}  // namespace

int fmoe_run_static_ws(const fmoe_traits_c* traits, const fmoe_args_c* args, void* stream) {
  int rc = validate_traits(traits);
  if (rc == FMOE_OK) rc = validate_dims(traits, args);
  if (rc != FMOE_OK) return rc;
  Plan plan;
  make_plan(traits, args, &plan);
  if (plan.l.total_bytes > static_cast<uint64_t>(FMOE_STATIC_WS_BYTES))
    return fail(FMOE_ERR_WORKSPACE,
                "this call needs %llu bytes of scratch but the built-in workspace holds %llu; "
                "use fmoe_run with a caller-provided workspace",
                (unsigned long long)plan.l.total_bytes, (unsigned long long)FMOE_STATIC_WS_BYTES);
  if (args->T > 0 && args->x) {
    rc = set_device_for(args->x);
    if (rc != FMOE_OK) return rc;
  }
  int dev = 0;
  FMOE_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kStaticWsMaxDevices) return fail(FMOE_ERR_UNSUPPORTED, "device index %d out of range", dev);
  void* ws = nullptr;
  {
    std::lock_guard<std::mutex> lock(g_static_ws_mu);
    if (g_static_ws_addr[dev] == nullptr) {
      // In host code the array's name is only a handle; the address kernels can use has to
      // be asked for, once per device, with that device current.
      void* p = nullptr;
      cudaError_t e = cudaGetSymbolAddress(&p, g_fmoe_static_ws);
      if (e != cudaSuccess || p == nullptr)
        return fail(FMOE_ERR_CUDA, "cudaGetSymbolAddress(static workspace) failed on device %d: %s", dev,
                    cudaGetErrorString(e));
      g_static_ws_addr[dev] = p;
    }
    ws = g_static_ws_addr[dev];
  }
  fmoe_args_c a = *args;
  a.workspace = ws;
  a.workspace_bytes = FMOE_STATIC_WS_BYTES;
  // The sorting kernel rewrites every word later kernels read (pad slots, block ids, the
  // status word), so nothing left over from the previous call needs clearing here.
  return run_impl(traits, &a, stream, nullptr, nullptr);
}

// ---- expert-parallel helpers: pack rows for the dispatch, reduce the returned rows.
int fmoe_gather_rows(const void* src, int32_t n_src, int32_t cols, const int32_t* row_ids, int32_t n_rows,
                     const int32_t* n_rows_dev, void* dst, void* stream) {
  if (!src || !row_ids || !dst || !n_rows_dev) return fail(FMOE_ERR_INVALID_ARG, "src, row_ids, n_rows_dev and dst are required");
  if (cols <= 0 || cols % 8) return fail(FMOE_ERR_UNSUPPORTED, "cols must be a positive multiple of 8");
  if (n_rows <= 0) return FMOE_OK;
  int rc = set_device_for(src);
  if (rc != FMOE_OK) return rc;
  FMOE_CUDA(fmoe::launch_gather_rows(src, n_src, cols, row_ids, n_rows_dev, n_rows, 0, dst, nullptr,
                                     static_cast<cudaStream_t>(stream)));
  return FMOE_OK;
}

int fmoe_combine_rows(const void* rows, const int32_t* index, int32_t T, int32_t K, int32_t H, void* out,
                      void* stream) {
  if (!rows || !index || !out) return fail(FMOE_ERR_INVALID_ARG, "rows, index and out are required");
  if (H <= 0 || H % 8) return fail(FMOE_ERR_UNSUPPORTED, "H must be a positive multiple of 8");
  if (T <= 0) return FMOE_OK;
  int rc = set_device_for(rows);
  if (rc != FMOE_OK) return rc;
  FMOE_CUDA(fmoe::launch_combine_rows(rows, index, T, K, H, out, static_cast<cudaStream_t>(stream)));
  return FMOE_OK;
}

int fmoe_check_status(const void* workspace, void* stream, int32_t* status_out) {
  if (!workspace || !status_out) return fail(FMOE_ERR_INVALID_ARG, "workspace and status_out are required");
  // the meta block is the first region of every workspace layout; word 1 is the status
  const int32_t* status = reinterpret_cast<const int32_t*>(workspace) + 1;
  FMOE_CUDA(cudaMemcpyAsync(status_out, status, sizeof(int32_t), cudaMemcpyDeviceToHost,
                            static_cast<cudaStream_t>(stream)));
  FMOE_CUDA(cudaStreamSynchronize(static_cast<cudaStream_t>(stream)));
  if (*status_out != 0) return fail(FMOE_ERR_DEVICE_TIMEOUT, "device status word 0x%x", *status_out);
  return FMOE_OK;
}

}  // extern "C"
