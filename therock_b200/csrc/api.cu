// C-ABI of libfmoe_b200.so: argument validation, workspace planning and the launch
// sequence of the fused-MoE operator.  No device memory is allocated here; every buffer
// belongs to the caller.
#include <cuda_runtime.h>
#include <nvtx3/nvToolsExt.h>

#include <cstdio>
#include <cstring>
#include <mutex>

#include "../../include/fused_moe_c.h"
#include "gemm.cuh"
#include "internal.h"
#include "plan.hpp"

namespace {

using fmoe::fail;
using fmoe::Plan;
using fmoe::make_plan;
using fmoe::validate_dims;
using fmoe::validate_traits;

// Makes the device that owns `ptr` current for the lifetime of the object and puts the
// caller's device back afterwards: the entry points leave no trace in the calling thread.
class DeviceGuard {
 public:
  explicit DeviceGuard(const void* ptr) {
    cudaPointerAttributes attr;
    if (ptr == nullptr || cudaPointerGetAttributes(&attr, ptr) != cudaSuccess) {
      cudaGetLastError();   // not fatal: stay on the calling thread's device
      return;
    }
    if (attr.type != cudaMemoryTypeDevice) return;
    int cur = -1;
    if (cudaGetDevice(&cur) != cudaSuccess || cur == attr.device) return;
    if (cudaSetDevice(attr.device) != cudaSuccess) {
      rc_ = fail(FMOE_ERR_CUDA, "cudaSetDevice(%d) failed", attr.device);
      return;
    }
    prev_ = cur;
  }
  ~DeviceGuard() {
    if (prev_ >= 0) cudaSetDevice(prev_);
  }
  DeviceGuard(const DeviceGuard&) = delete;
  DeviceGuard& operator=(const DeviceGuard&) = delete;
  int rc() const { return rc_; }

 private:
  int prev_ = -1;
  int rc_ = FMOE_OK;
};

// A pair of timing events that is destroyed on every exit path.
struct EventPair {
  cudaEvent_t a = nullptr, b = nullptr;
  ~EventPair() {
    if (a) cudaEventDestroy(a);
    if (b) cudaEventDestroy(b);
  }
};

// NVTX range around one stage of the operator (a no-op unless a profiler is attached).
struct NvtxRange {
  explicit NvtxRange(const char* name) { nvtxRangePushA(name); }
  ~NvtxRange() { nvtxRangePop(); }
};

#define FMOE_CUDA(expr)                                                                    \
  do {                                                                                     \
    cudaError_t e__ = (expr);                                                              \
    if (e__ != cudaSuccess)                                                                \
      return fail(FMOE_ERR_CUDA, "%s failed: %s", #expr, cudaGetErrorString(e__));         \
  } while (0)

}  // namespace

extern "C" {

int fmoe_version(void) { return 100; }

const char* fmoe_last_error(void) { return fmoe::last_error_buf(); }

int64_t fmoe_sort_capacity(int32_t T, int32_t K, int32_t E, int32_t block_m) {
  return fmoe::sort_capacity(T, K, E, block_m);
}

int fmoe_sort(const int32_t* topk_ids, const float* topk_weight, int32_t T, int32_t K, int32_t E,
              int32_t block_m, int32_t* sorted_token_ids, float* sorted_weights,
              int32_t* sorted_expert_ids, int32_t* num_tokens_post_pad, void* stream) {
  if (!topk_ids || !sorted_token_ids) return fail(FMOE_ERR_INVALID_ARG, "topk_ids and sorted_token_ids are required");
  if (sorted_weights && !topk_weight) return fail(FMOE_ERR_INVALID_ARG, "sorted_weights requested without topk_weight");
  if (T < 0 || K <= 0 || E <= 0 || block_m <= 0) return fail(FMOE_ERR_INVALID_ARG, "bad dimensions");
  if (E > 1024) return fail(FMOE_ERR_UNSUPPORTED, "at most 1024 experts");
  if (static_cast<int64_t>(T) * K > (1 << 24)) return fail(FMOE_ERR_UNSUPPORTED, "T*K too large");
  DeviceGuard guard(topk_ids);
  if (guard.rc() != FMOE_OK) return guard.rc();
  NvtxRange range("fmoe_sort");
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

int fmoe_describe_run(const fmoe_traits_c* traits, const fmoe_args_c* args, fmoe_run_info_c* info) {
  int rc = validate_traits(traits);
  if (rc == FMOE_OK) rc = validate_dims(traits, args);
  if (rc != FMOE_OK) return rc;
  if (!info) return fail(FMOE_ERR_INVALID_ARG, "info is null");
  *info = fmoe_run_info_c{};
  const int forced = traits->gemm_mode ? traits->gemm_mode : fmoe::gemm_mode_override();
  return fmoe::describe_run(traits, args, fmoe::device_sm_count(), forced, info);
}

const char* fmoe_gemm_kernel_name(int32_t kernel) {
  switch (kernel) {
    case FMOE_KERNEL_SINGLE: return "fmoe_grouped_gemm_kernel";
    case FMOE_KERNEL_PAIR: return "fmoe_grouped_gemm_pair_kernel";
    case FMOE_KERNEL_BLOCK_PROMOTE: return "fmoe_grouped_gemm_block_kernel<promote>";
    case FMOE_KERNEL_BLOCK_HW_SCALE: return "fmoe_grouped_gemm_block_kernel<block_scale MMA>";
    case FMOE_KERNEL_SINGLE_DECODE: return "fmoe_grouped_gemm_kernel<32 activation rows>";
    case FMOE_KERNEL_BLOCK_HW_TOKENS_N: return "fmoe_grouped_gemm_tokn_kernel";
    default: return "";
  }
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
  const bool fp8 = fmoe::quant_is_fp8(traits->quant);
  if (!a.x || !a.w1 || !a.w2 || !a.topk_ids || !a.topk_weight || (!a.out && !a.partial_row_ptrs))
    return fail(FMOE_ERR_INVALID_ARG, "x, w1, w2, topk_ids, topk_weight and out are required");
  if (fp8 && (!a.w1_scale || !a.w2_scale)) return fail(FMOE_ERR_INVALID_ARG, "fp8 variants need w1_scale and w2_scale");
  if (a.partial_row_ptrs && traits->partial_dtype != FMOE_PARTIAL_BF16)
    return fail(FMOE_ERR_INVALID_ARG, "partial_row_ptrs needs partial_dtype = bf16");
  if (a.done_flag_addrs && (!a.partial_row_ptrs || !a.done_flag_value || !a.done_counter || a.done_flag_count <= 0))
    return fail(FMOE_ERR_INVALID_ARG, "done_flag_addrs needs partial_row_ptrs, done_flag_value, done_counter and a positive count");
  Plan plan;
  make_plan(traits, args, &plan);
  if (!a.workspace) return fail(FMOE_ERR_WORKSPACE, "workspace is null (%llu bytes needed)", (unsigned long long)plan.l.total_bytes);
  if (a.workspace_bytes < plan.l.total_bytes)
    return fail(FMOE_ERR_WORKSPACE, "workspace has %llu bytes, %llu needed", (unsigned long long)a.workspace_bytes,
                (unsigned long long)plan.l.total_bytes);
  if (reinterpret_cast<uintptr_t>(a.workspace) & 255) return fail(FMOE_ERR_WORKSPACE, "workspace must be 256-byte aligned");

  DeviceGuard guard(a.x);
  if (guard.rc() != FMOE_OK) return guard.rc();
  NvtxRange whole("fmoe_run");

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
  void* a_scale = fp8 ? ws + l.a_scale : nullptr;
  void* y = ws + l.y;
  void* yq = ws + l.y_quant;
  void* y_scale = fp8 ? ws + l.y_scale : nullptr;
  void* slots = ws + l.slots;

#define FMOE_STAGE(i) do { if (stage_ev) FMOE_CUDA(cudaEventRecord(stage_ev[i], stream)); } while (0)
  EventPair ev;
  FMOE_STAGE(0);
  if (ms_out) {
    FMOE_CUDA(cudaEventCreate(&ev.a));
    FMOE_CUDA(cudaEventCreate(&ev.b));
    FMOE_CUDA(cudaEventRecord(ev.a, stream));
  }

  const bool blk = fmoe::quant_is_block(traits->quant);
  const bool hw = traits->quant == FMOE_QUANT_BLOCK128_UE8M0;
  const int qmode = !fp8 ? 0 : (hw ? 3 : (blk ? 2 : 1));
  if (a.x_scale == nullptr && fmoe::decode_prologue_applies(a.T, a.K, qmode)) {
    // decode-sized batch: sorting and gather (+ quantisation) are one launch
    NvtxRange r("decode_prologue");
    FMOE_CUDA(fmoe::launch_decode_prologue(a.topk_ids, a.topk_weight, a.T, a.K, a.E, plan.cap, a.x, a.H, qmode,
                                           sorted_ids, sorted_w, sorted_rows, expert_ids, num_post_pad, mblk_cum,
                                           status, a_sorted, static_cast<float*>(a_scale), stream, a.num_tokens_dev));
    FMOE_STAGE(1);
  } else {
    {
      NvtxRange r("moe_sorting");
      FMOE_CUDA(fmoe::launch_moe_sorting(a.topk_ids, a.topk_weight, a.T, a.K, a.E, traits->block_m, plan.cap,
                                         sorted_ids, sorted_w, sorted_rows, expert_ids, num_post_pad,
                                         mblk_cum, status, stream, a.num_tokens_dev, 1, nullptr,
                                         reinterpret_cast<int32_t*>(ws + l.sort_scratch)));
    }
    FMOE_STAGE(1);
    NvtxRange r("gather_quant");
    if (a.x_scale != nullptr) {
      // the caller's rows are e4m3 with their scales already: the routed pairs copy them
      FMOE_CUDA(fmoe::launch_gather_quantised(a.x, a.x_scale, a.T, a.H, sorted_ids, num_post_pad, plan.cap, qmode,
                                              a_sorted, a_scale, stream));
    } else if (fmoe::quantise_once(traits, args)) {
      // every token row is quantised once; the routed pairs then copy e4m3 rows and scales
      void* xq = ws + l.x_quant;
      void* xq_scale = ws + l.x_quant_scale;
      FMOE_CUDA(fmoe::launch_gather_rows(a.x, a.T, a.H, nullptr, a.num_tokens_dev, a.T, qmode, xq, xq_scale, stream));
      FMOE_CUDA(fmoe::launch_gather_quantised(xq, xq_scale, a.T, a.H, sorted_ids, num_post_pad, plan.cap, qmode,
                                              a_sorted, a_scale, stream));
    } else {
      FMOE_CUDA(fmoe::launch_gather_rows(a.x, a.T, a.H, sorted_ids, num_post_pad, plan.cap, qmode,
                                         a_sorted, a_scale, stream, nullptr, /*skip_pad=*/true));
    }
  }
  FMOE_STAGE(2);

  fmoe::GemmLaunch g{};
  int drv = 0;
  g.fp8 = fp8;
  g.b_tiled = traits->weight_layout == FMOE_WEIGHTS_TILED128;
  g.num_experts = a.E;
  g.mblk_cum = mblk_cum;
  g.sorted_rows = sorted_rows;
  g.sorted_weights = sorted_w;
  g.status = status;
  g.max_m_blocks = static_cast<int>(plan.cap / fmoe::kBlockM);
  const int forced_mode = traits->gemm_mode ? traits->gemm_mode : fmoe::gemm_mode_override();
  const int sms = fmoe::device_sm_count();
  const bool fused_quant = blk && fmoe::kFusedBlockQuant;
  // gemm1: [cap, H] x W1[E, 2I, H]^T -> SiLU(gate) * up -> y [cap, I]
  if (traits->gate_only) {
    // W1 is [E, I, H]: a tile is 256 consecutive gate rows, y = SiLU(gate)
    g.epilogue = fmoe::kEpiSilu;
    g.b_rows_per_expert = a.I;
    g.n_blocks = a.I / fmoe::kTileN; g.n_stride = fmoe::kTileN; g.second_slab_offset = fmoe::kSlabRows;
  } else {
    g.epilogue = fmoe::kEpiSiluMul;
    g.b_rows_per_expert = 2 * a.I;
    g.n_blocks = a.I / fmoe::kSlabRows; g.n_stride = fmoe::kSlabRows; g.second_slab_offset = a.I;
  }
  g.flavour = fmoe::pick_gemm_flavour(traits, args, g.n_blocks, sms, forced_mode);
  g.a = a_sorted; g.a_rows = plan.cap; g.b = a.w1; g.k_elems = a.H;
  g.a_scale = a_scale; g.b_scale = fp8 ? a.w1_scale : nullptr;
  g.out = fused_quant ? yq : y; g.ld_out = a.I;
  g.out_rows = plan.cap;
  g.out_scale = fused_quant ? y_scale : nullptr;
  {
    NvtxRange r("gemm1_silu_mul");
    if (fmoe::launch_grouped_gemm(g, stream, &drv) != cudaSuccess)
      return fail(FMOE_ERR_CUDA, "gemm1 launch failed (cuda: %s, driver code %d)", cudaGetErrorString(cudaGetLastError()), drv);
  }
  FMOE_STAGE(3);

  const void* a2 = y;
  if (fp8) {
    if (!fused_quant) {
      NvtxRange r("quant_intermediate");
      FMOE_CUDA(fmoe::launch_gather_rows(y, static_cast<int>(plan.cap), a.I, nullptr, num_post_pad, plan.cap, qmode,
                                         yq, y_scale, stream, sorted_rows));
    }
    a2 = yq;
  }
  FMOE_STAGE(4);
  // gemm2: [cap, I] x W2[E, H, I]^T * topk_weight -> slots [T*K, H]
  g.epilogue = fmoe::kEpiScaledSlots;
  g.a = a2; g.b = a.w2; g.k_elems = a.I;
  g.b_rows_per_expert = a.H;
  g.n_blocks = a.H / fmoe::kTileN; g.n_stride = fmoe::kTileN; g.second_slab_offset = fmoe::kSlabRows;
  g.flavour = fmoe::pick_gemm_flavour(traits, args, g.n_blocks, sms, forced_mode);
  g.a_scale = y_scale; g.b_scale = fp8 ? a.w2_scale : nullptr;
  g.out = slots; g.ld_out = a.H;
  g.out_rows = static_cast<int64_t>(a.T) * a.K;
  g.out_scale = nullptr;
  g.out_bf16 = traits->partial_dtype == FMOE_PARTIAL_BF16;
  g.row_ptrs = a.partial_row_ptrs;
  g.done_addrs = a.done_flag_addrs;
  g.done_value = a.done_flag_value;
  g.done_counter = a.done_counter;
  g.done_count = a.done_flag_count;
  {
    NvtxRange r("gemm2_weighted");
    if (fmoe::launch_grouped_gemm(g, stream, &drv) != cudaSuccess)
      return fail(FMOE_ERR_CUDA, "gemm2 launch failed (cuda: %s, driver code %d)", cudaGetErrorString(cudaGetLastError()), drv);
  }
  FMOE_STAGE(5);

  if (!a.partial_row_ptrs) {    // scattered partial rows are added up by their owner
    NvtxRange r("combine");
    FMOE_CUDA(fmoe::launch_combine(slots, g.out_bf16, a.topk_ids, a.T, a.K, a.E, a.H, a.out, stream, a.num_tokens_dev));
  }
  FMOE_STAGE(6);
#undef FMOE_STAGE

  if (ms_out) {
    FMOE_CUDA(cudaEventRecord(ev.b, stream));
    FMOE_CUDA(cudaEventSynchronize(ev.b));
    FMOE_CUDA(cudaEventElapsedTime(ms_out, ev.a, ev.b));
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
    if (cudaEventCreate(&p->ev[i]) != cudaSuccess) {
      for (int j = 0; j < i; ++j) cudaEventDestroy(p->ev[j]);
      delete[] p->ev;
      delete p;
      return fail(FMOE_ERR_CUDA, "cudaEventCreate failed");
    }
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
  DeviceGuard guard(args->T > 0 ? args->x : nullptr);
  if (guard.rc() != FMOE_OK) return guard.rc();
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
  // The first kernel rewrites every index, count and status word later kernels act on (sorted
  // ids, block table, pad markers).  Activation rows of pad slots may hold what an earlier call
  // left there: the GEMMs multiply them, but rows without a token are never stored, so nothing
  // needs clearing here.
  return run_impl(traits, &a, stream, nullptr, nullptr);
}

// ---- expert-parallel helpers: pack rows for the dispatch, reduce the returned rows.
int fmoe_gather_rows(const void* src, int32_t n_src, int32_t cols, const int32_t* row_ids, int32_t n_rows,
                     const int32_t* n_rows_dev, void* dst, void* stream) {
  if (!src || !row_ids || !dst || !n_rows_dev) return fail(FMOE_ERR_INVALID_ARG, "src, row_ids, n_rows_dev and dst are required");
  if (cols <= 0 || cols % 8) return fail(FMOE_ERR_UNSUPPORTED, "cols must be a positive multiple of 8");
  if (n_rows <= 0) return FMOE_OK;
  DeviceGuard guard(src);
  if (guard.rc() != FMOE_OK) return guard.rc();
  FMOE_CUDA(fmoe::launch_gather_rows(src, n_src, cols, row_ids, n_rows_dev, n_rows, 0, dst, nullptr,
                                     static_cast<cudaStream_t>(stream)));
  return FMOE_OK;
}

int fmoe_quantise_rows(const void* x, int32_t T, int32_t H, int32_t quant, void* q, void* scales, void* stream) {
  if (!x || !q || !scales) return fail(FMOE_ERR_INVALID_ARG, "x, q and scales are required");
  if (quant != FMOE_QUANT_TOKEN_CHANNEL && quant != FMOE_QUANT_BLOCK128 && quant != FMOE_QUANT_BLOCK128_UE8M0)
    return fail(FMOE_ERR_INVALID_ARG, "quant must be an fp8 mode");
  if (H <= 0 || H % 16 || (quant != FMOE_QUANT_TOKEN_CHANNEL && H % 128))
    return fail(FMOE_ERR_UNSUPPORTED, "H must be a multiple of 16 (128 for the block modes)");
  if (T <= 0) return FMOE_OK;
  DeviceGuard guard(x);
  if (guard.rc() != FMOE_OK) return guard.rc();
  const int qmode = quant == FMOE_QUANT_TOKEN_CHANNEL ? 1 : (quant == FMOE_QUANT_BLOCK128 ? 2 : 3);
  FMOE_CUDA(fmoe::launch_gather_rows(x, T, H, nullptr, nullptr, T, qmode, q, scales, static_cast<cudaStream_t>(stream)));
  return FMOE_OK;
}

int fmoe_combine_rows(const void* rows, const int32_t* index, int32_t T, int32_t K, int32_t H, void* out,
                      void* stream) {
  if (!rows || !index || !out) return fail(FMOE_ERR_INVALID_ARG, "rows, index and out are required");
  if (H <= 0 || H % 8) return fail(FMOE_ERR_UNSUPPORTED, "H must be a positive multiple of 8");
  if (T <= 0) return FMOE_OK;
  DeviceGuard guard(rows);
  if (guard.rc() != FMOE_OK) return guard.rc();
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
