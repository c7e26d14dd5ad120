/*
 * C-ABI of the B200 fused-MoE library (libfmoe_b200.so).
 *
 * This is the boundary a foreign-function binding attaches to: plain C structs with
 * fixed-width integers, device pointers as void*, the CUDA stream as void*.  No C++
 * or torch types appear in any signature.
 *
 * What it replaces: Composable Kernel's ck_tile fused-MoE host entry points
 * (fused_moe_traits / fused_moe_args / fused_moe(traits, args, stream) and the separately
 * callable moe_sorting).  TheRock builds that library from the rocm-libraries submodule
 * (math-libs/CMakeLists.txt:582-608, source dir projects/composablekernel; submodule
 * declared at .gitmodules:19-22) and ships only include/ck/** for it
 * (math-libs/artifact-composable-kernel.toml:5-8).  The submodule is empty in the
 * reference checkout, so no file:line inside the ck_tile headers can be cited; the C++
 * mirror of the host surface is include/fused_moe.hpp.
 *
 * Ownership: the caller owns every device buffer, including the workspace whose size is
 * queried with fmoe_get_workspace_size.  The library allocates no device memory.
 * Errors: every entry point returns 0 on success or a negative fmoe_status; the text of
 * the last error on the calling thread is available from fmoe_last_error().  Nothing
 * throws across this boundary and no device code traps.
 */
#ifndef FMOE_B200_FUSED_MOE_C_H_
#define FMOE_B200_FUSED_MOE_C_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define FMOE_API __attribute__((visibility("default")))
#else
#define FMOE_API
#endif

enum fmoe_status {
  FMOE_OK = 0,
  FMOE_ERR_INVALID_ARG = -1,    /* null pointer, bad dimension, unsupported combination */
  FMOE_ERR_UNSUPPORTED = -2,    /* shape / dtype / block size outside what the kernels tile */
  FMOE_ERR_WORKSPACE = -3,      /* workspace pointer missing or too small */
  FMOE_ERR_CUDA = -4,           /* a CUDA runtime / driver call failed */
  FMOE_ERR_DEVICE_TIMEOUT = -5  /* a bounded device-side wait ran out (status word set) */
};

enum fmoe_dtype { FMOE_BF16 = 0, FMOE_FP8_E4M3 = 1 };

enum fmoe_quant {
  FMOE_QUANT_NONE = 0,          /* bf16 activations and weights */
  FMOE_QUANT_TOKEN_CHANNEL = 1, /* fp8: dynamic per-token activation scale, per-output-channel weight scale */
  FMOE_QUANT_BLOCK128 = 2,      /* fp8: 1x128 activation groups, 128x128 weight blocks, f32 scales */
  FMOE_QUANT_BLOCK128_UE8M0 = 3 /* same granularity with power-of-two scales (the MX "UE8M0" scale format):
                                   activation scales are 2^ceil(log2(absmax/448)); the weight scales passed
                                   in must be powers of two.  The scales are applied inside the tensor core
                                   (tcgen05.mma kind::mxf8f6f4.block_scale), the accumulator never leaves
                                   tensor memory during the K loop */
};

/* How the K weighted expert outputs of a token are held before the ordered sum. */
enum fmoe_partial_dtype {
  FMOE_PARTIAL_F32 = 0, /* f32: out = bf16( sum_k f32 partial ), one rounding (the default contract) */
  FMOE_PARTIAL_BF16 = 1 /* each partial is rounded to bf16 first, then summed in f32 in k order and rounded
                           once more: halves the traffic of the partial rows; this is also what the
                           expert-parallel path does, where partial rows cross NVLink as bf16 */
};

/* Kernel flavours of the grouped GEMM, as reported by fmoe_describe_run. */
enum fmoe_gemm_kernel {
  FMOE_KERNEL_SINGLE = 1,        /* fmoe_grouped_gemm_kernel: one CTA per 128 x 256 tile */
  FMOE_KERNEL_PAIR = 2,          /* fmoe_grouped_gemm_pair_kernel: CTA pair, cta_group::2, 256 x 256 tile */
  FMOE_KERNEL_BLOCK_PROMOTE = 3, /* fmoe_grouped_gemm_block_kernel<.., false>: per-128 partials promoted in registers */
  FMOE_KERNEL_BLOCK_HW_SCALE = 4,/* fmoe_grouped_gemm_block_kernel<.., true>: block_scale MMA, UE8M0 scales */
  FMOE_KERNEL_SINGLE_DECODE = 5, /* fmoe_grouped_gemm_kernel staging 32 activation rows (at most 32 routed rows) */
  FMOE_KERNEL_BLOCK_HW_TOKENS_N = 6 /* fmoe_grouped_gemm_tokn_kernel: block_scale MMA with the weights on M and
                                       the tokens on N in steps of 16, so padding rows are not multiplied */
};

enum fmoe_activation { FMOE_ACT_SILU = 0 };

enum fmoe_weight_layout {
  FMOE_WEIGHTS_ROW_MAJOR = 0, /* [E, rows, K], K contiguous */
  FMOE_WEIGHTS_TILED128 = 1   /* pre-shuffled: [E, rows/128, K_bytes/128, 128 rows, 128 bytes] -- every
                                 128-row x 128-byte operand tile is one contiguous 16 KiB block, so the
                                 weight stream reads DRAM in long bursts (same values, same results) */
};

/* Compile-time-like selection of the operator variant (ck_tile's fused_moe_traits role). */
typedef struct fmoe_traits_c {
  int32_t quant;        /* fmoe_quant */
  int32_t weight_dtype; /* fmoe_dtype; must agree with quant */
  int32_t activation;   /* fmoe_activation */
  int32_t gate_only;    /* 0: W1 holds gate rows then up rows [E,2I,H], y = SiLU(gate)*up;
                           1: W1 is [E,I,H] and y = SiLU(gate) (I a multiple of 256; not with block128) */
  int32_t block_m;      /* rows per sorted block; 128 */
  int32_t gemm_mode;    /* 0 = chosen per GEMM from the expected tile counts, 1 = single-CTA
                           kernel, 2 = CTA-pair kernel (cta_group::2); with block128_ue8m0:
                           0 and 1 = tokens on M (128-row blocks), 2 = tokens on N (steps of 16;
                           measured slower on the shapes benchmarked, kept selectable) */
  int32_t weight_layout; /* fmoe_weight_layout of w1 and w2 */
  int32_t partial_dtype; /* fmoe_partial_dtype */
} fmoe_traits_c;

/* Run-time arguments (ck_tile's fused_moe_args role).  All pointers are device pointers. */
typedef struct fmoe_args_c {
  const void* x;            /* [T, H] bf16 activations ([T, H] e4m3 when x_scale is set) */
  const void* w1;           /* [E, 2I, H] gate rows then up rows ([E, I, H] when gate_only); bf16 or e4m3 */
  const void* w2;           /* [E, H, I]; bf16 or e4m3 */
  const float* w1_scale;    /* quant 1: [E, 2I]; quant 2, 3: [E, 2I/128, H/128]; else NULL */
  const float* w2_scale;    /* quant 1: [E, H];  quant 2, 3: [E, H/128, I/128]; else NULL */
  const int32_t* topk_ids;  /* [T, K]; ids outside [0, E) are skipped */
  const float* topk_weight; /* [T, K] */
  void* out;                /* [T, H] bf16 */
  void* workspace;          /* >= fmoe_get_workspace_size bytes, 256-byte aligned */
  uint64_t workspace_bytes;
  int32_t T, H, I, E, K;
  int32_t expected_tokens;  /* 0, or the token count the caller expects when T is only a capacity
                               (see num_tokens_dev): used to pick the GEMM kernel flavour */
  int32_t reserved[2];
  const int32_t* num_tokens_dev; /* optional device int32: only the first min(T, *num_tokens_dev)
                                    tokens are processed (T still sizes the workspace); used when
                                    the batch size is only known on the device, e.g. on the
                                    receiving side of an expert-parallel dispatch.  NULL = T. */
  /* Scattered partial rows (optional; expert parallelism).  When set, traits.partial_dtype must
   * be bf16, the weighted output row of routed pair (t, k) is stored as bf16 at the device
   * address partial_row_ptrs[t*K + k] (which may lie in a peer GPU's memory: plain stores), `out`
   * is not written and no combine runs -- whoever owns those rows adds them up
   * (fmoe_ep_wait_combine).  Entries of pairs whose expert id is outside [0, E) are not read. */
  const uint64_t* partial_row_ptrs;
  /* Completion signal (optional; used with partial_row_ptrs).  When the last CTA of the second
   * GEMM has stored its rows it writes *done_flag_value, with release semantics at system scope,
   * to each of the done_flag_count addresses in done_flag_addrs (a device array; the addresses
   * may be peer memory), so a consumer on another GPU can wait for the rows without another
   * kernel launch.  done_counter is one zero-initialised device int32 the library uses to find
   * the last CTA; it is left at zero. */
  const uint64_t* done_flag_addrs;
  const int32_t* done_flag_value;
  int32_t* done_counter;
  int32_t done_flag_count;
  int32_t reserved2;
  /* Activations that are already quantised (optional; fp8 quant modes only).  When set, x holds
   * e4m3 rows and x_scale their scales exactly as fmoe_quantise_rows writes them for traits.quant
   * (f32 [T], f32 [T, H/128] or UE8M0 bytes [T, roundup(H/128, 4)]); the operator skips its own
   * quantisation of x and the result is bit-identical to passing the bf16 rows.  Used on the
   * receiving side of an expert-parallel dispatch that sends e4m3 rows. */
  const void* x_scale;
} fmoe_args_c;

/* Library version: major*10000 + minor*100 + patch. */
FMOE_API int fmoe_version(void);

/* Text of the most recent error on the calling thread ("" if none). */
FMOE_API const char* fmoe_last_error(void);

/* Capacity (in slots) of the sorted arrays for T tokens, K experts per token, E experts:
 * T*K + E*(block_m-1) rounded up to block_m. */
FMOE_API int64_t fmoe_sort_capacity(int32_t T, int32_t K, int32_t E, int32_t block_m);

/* moe_sorting: stable bucket of the T*K (token, k) pairs by expert id, each bucket padded
 * to a multiple of block_m.  Outputs (device): sorted_token_ids[cap] (pad = T),
 * sorted_weights[cap] (pad = 0), sorted_expert_ids[cap/block_m] (unused blocks = -1),
 * num_tokens_post_pad[1].  Enqueues on `stream` and returns.
 * Replaces ck_tile's moe_sorting host call (source absent from the reference checkout). */
FMOE_API int fmoe_sort(const int32_t* topk_ids, const float* topk_weight, int32_t T, int32_t K,
                       int32_t E, int32_t block_m, int32_t* sorted_token_ids,
                       float* sorted_weights, int32_t* sorted_expert_ids,
                       int32_t* num_tokens_post_pad, void* stream);

/* Router: logits [T, E] f32 -> topk_ids [T, K] int32, topk_weight [T, K] f32 on the device.
 * mode 0 = softmax over the experts, 1 = sigmoid; the K best scores are kept (ties to the
 * lower expert index) and divided by their sum.  E <= 1024, K <= 32.  This is the input
 * preparation the ck_tile example drivers do on the host before calling fused_moe; here it
 * is a kernel so logits -> fused_moe needs no host step. */
FMOE_API int fmoe_route(const float* logits, int32_t T, int32_t E, int32_t K, int32_t mode,
                        int32_t* topk_ids, float* topk_weight, void* stream);

/* Byte offsets of the regions fmoe_run keeps in the workspace.  After a run has completed
 * the regions hold that run's intermediates, which lets a caller (or a test) inspect every
 * stage: meta[0] = num_tokens_post_pad, meta[1] = device status word. */
typedef struct fmoe_ws_layout_c {
  int64_t capacity;           /* slots in the sorted arrays */
  uint64_t total_bytes;
  uint64_t meta;              /* int32[64] */
  uint64_t sorted_token_ids;  /* int32[capacity] */
  uint64_t sorted_weights;    /* float[capacity] */
  uint64_t sorted_rows;       /* int32[capacity]: flat token*K+k per slot, -1 = pad */
  uint64_t sorted_expert_ids; /* int32[capacity/block_m] */
  uint64_t mblk_cum;          /* int32[E+1]: cumulative blocks per expert */
  uint64_t a_sorted;          /* [capacity, H] activations in sorted order (bf16 or e4m3) */
  uint64_t a_scale;           /* quant 1: float[capacity]; quant 2: float[capacity, H/128]; quant 3: one UE8M0
                                 byte (biased exponent) per row and 128-wide K group, row-major, rows
                                 padded to a multiple of four bytes */
  uint64_t y;                 /* bf16 [capacity, I]: SiLU(gate)*up (quant 0, 1; the block-scaled modes
                                 quantise inside the first GEMM and keep no bf16 copy) */
  uint64_t y_quant;           /* e4m3 [capacity, I] (fp8 variants) */
  uint64_t y_scale;           /* as a_scale, with I in place of H */
  uint64_t slots;             /* float or bf16 (traits.partial_dtype) [T*K, H]: weighted expert outputs */
  uint64_t sort_scratch;      /* int32[128*E]: per-CTA histograms of the multi-CTA moe_sorting */
  uint64_t x_quant;           /* e4m3 [T, H]: the token rows quantised once (fp8 variants with K >= 2, not
                                 decode-sized); a_sorted is then gathered from here */
  uint64_t x_quant_scale;     /* their scales, laid out as a_scale with T rows */
} fmoe_ws_layout_c;

FMOE_API int fmoe_get_workspace_layout(const fmoe_traits_c* traits, const fmoe_args_c* args,
                                       fmoe_ws_layout_c* layout);

/* Bytes of workspace fmoe_run needs for these traits / dimensions. */
FMOE_API int fmoe_get_workspace_size(const fmoe_traits_c* traits, const fmoe_args_c* args,
                                     uint64_t* bytes);

/* The fused operator: moe_sorting -> gather(+quant) -> gemm1 + SiLU*up -> (quant) ->
 * gemm2 * topk_weight -> ordered combine into out.  Asynchronous on `stream` when ms_out
 * is NULL; when ms_out is given the call synchronises and stores the elapsed milliseconds.
 * Replaces ck_tile's fused_moe(traits, args, stream). */
FMOE_API int fmoe_run(const fmoe_traits_c* traits, const fmoe_args_c* args, void* stream,
                      float* ms_out);

/* fmoe_run for callers that cannot allocate device memory (no counterpart in the reference:
 * ck_tile always takes its workspace from the caller).  Meant for hosts that receive only
 * input and output buffers -- a plugin slot of a serving engine, a foreign-function caller
 * without a CUDA allocator, a loop where cudaMalloc is forbidden because it stalls the
 * device.  Inputs and outputs are passed as for fmoe_run; args->workspace is ignored and
 * the scratch comes from an array of FMOE_STATIC_WS_BYTES built into the library (each GPU
 * that loads the library holds that much until the process ends).  Calls whose workspace
 * (fmoe_get_workspace_size) exceeds the limit return FMOE_ERR_WORKSPACE.  The call itself
 * performs no cudaMalloc / cudaFree and uses no allocating library routine.
 * The first call on each device looks up the array's device address; make that first
 * call outside any stream capture.  All calls on a device share the one array and it keeps
 * the previous call's contents (every index and count later stages act on is rewritten by the
 * call's first kernel; stale activation rows of padding slots only feed results that are never
 * stored), so two calls that may overlap on the GPU -- different streams, or
 * different threads -- race: serialise them on one stream.  Asynchronous on `stream`.
 * The status word of a bounded device wait is not readable through this variant; use
 * fmoe_run with fmoe_check_status where that is needed. */
#define FMOE_STATIC_WS_BYTES (64u * 1024u * 1024u)
FMOE_API int fmoe_run_static_ws(const fmoe_traits_c* traits, const fmoe_args_c* args, void* stream);

/* Reads the device status word of a workspace after the stream has been synchronised:
 * 0 = clean, otherwise the code a kernel stored when a bounded wait ran out. */
FMOE_API int fmoe_check_status(const void* workspace, void* stream, int32_t* status_out);

/* Per-stage timing without synchronising inside the timed loop.  fmoe_profile_create
 * makes a handle holding events for up to max_runs runs; fmoe_run_profiled is fmoe_run
 * plus one event record between consecutive kernels; fmoe_profile_read waits for the
 * recorded runs, adds up the milliseconds of each of the six stages (sort, gather(+quant),
 * gemm1, quant of the intermediate, gemm2, combine) into stage_ms[6], stores the number of
 * runs and empties the handle.  No counterpart in ck_tile (its host API times the whole
 * call only). */
FMOE_API int fmoe_profile_create(int32_t max_runs, void** handle);
FMOE_API int fmoe_run_profiled(const fmoe_traits_c* traits, const fmoe_args_c* args, void* stream,
                               void* handle);
FMOE_API int fmoe_profile_read(void* handle, float* stage_ms, int32_t* runs);
FMOE_API int fmoe_profile_destroy(void* handle);

/* Expert-parallel pack: dst[i, :] = src[row_ids[i], :] for i < *n_rows_dev (a device
 * int32, <= n_rows); bf16 rows of `cols` elements; ids outside [0, n_src) give zero rows.
 * Used to lay token rows out per destination rank before the all-to-all dispatch.  The
 * reference operator is single-GPU (no counterpart); expert parallelism is added here. */
FMOE_API int fmoe_gather_rows(const void* src, int32_t n_src, int32_t cols, const int32_t* row_ids,
                              int32_t n_rows, const int32_t* n_rows_dev, void* dst, void* stream);

/* The operator's dynamic quantisation of activation rows as a call of its own: q[t, :] =
 * e4m3(x[t, :] / scale) with one scale per row (quant = token_channel: scales f32 [T]) or per
 * 128 columns (block128: f32 [T, H/128]; block128_ue8m0: power-of-two scales as bytes
 * [T, roundup(H/128, 4)]).  H a multiple of 16 (128 for the block modes).  No counterpart in the
 * reference operator, which quantises inside the call. */
FMOE_API int fmoe_quantise_rows(const void* x, int32_t T, int32_t H, int32_t quant, void* q, void* scales,
                                void* stream);

/* Expert-parallel combine: out[t, :] = bf16( sum over k ascending of rows[index[t*K+k], :] )
 * with f32 accumulation; index < 0 skips the term.  rows are the bf16 partial results that
 * came back through the all-to-all.  No counterpart in the single-GPU reference. */
FMOE_API int fmoe_combine_rows(const void* rows, const int32_t* index, int32_t T, int32_t K,
                               int32_t H, void* out, void* stream);

/* ---- Expert parallelism over peer memory (one process per GPU; no counterpart in the
 * single-GPU reference operator).  Every rank holds one buffer of identical layout that all
 * ranks of the node can address (peer_base[r] = address of rank r's buffer in this process,
 * a device array of G entries).  All calls are asynchronous on `stream`; none synchronises
 * with the host. */
typedef struct fmoe_ep_layout_c {
  uint64_t flags;    /* int32[G]: barrier epochs written by the peers */
  uint64_t matrix;   /* int32[G*G]: matrix[s*G+d] = rows rank s sends to rank d this step */
  uint64_t rows;     /* bf16 [recv_cap, H]: received token rows */
  uint64_t ids;      /* int32[recv_cap]: local expert id of each received row */
  uint64_t weights;  /* float[recv_cap]: routing weight of each received row */
  uint64_t src;      /* int32[recv_cap][2]: (source rank, source send slot) */
  uint64_t back;     /* bf16 [send_cap, H]: expert outputs returned to this rank */
  int64_t recv_cap;  /* rows the receive arrays hold (>= all routed pairs of the step) */
  int64_t send_cap;  /* rows of `back` (>= T*K of this rank) */
  uint64_t flags_dispatch; /* int32[G]: epoch at which each peer finished writing its rows here (fused path) */
  uint64_t flags_return;   /* int32[G]: epoch at which each peer finished returning this rank's rows (fused path) */
  uint64_t row_scales;     /* bytes [recv_cap, scale_row_bytes]: scales of the received rows when they travel as
                              e4m3 (fmoe_ep_send_rows); unused otherwise */
  uint64_t src_rank;       /* int32[recv_cap]: source rank of each received row (de-duplicated step, where
                              ids / weights are [recv_cap, K] and src is int32 [recv_cap, K]: pair index or -1) */
} fmoe_ep_layout_c;

/* Groups this rank's T*K routed pairs by the rank that owns the expert (stable):
 * order[i] = flat pair index of send slot i, inv_index[pair] = its slot (-1 if dropped),
 * cum[G+1] = cumulative rows per destination.  scratch_tokens: int32[T*K]. */
FMOE_API int fmoe_ep_plan(const int32_t* topk_ids, int32_t T, int32_t K, int32_t experts_per_rank,
                          int32_t G, int32_t* order, int32_t* inv_index, int32_t* cum,
                          int32_t* scratch_tokens, void* stream);
/* Writes this rank's row of the count matrix into every rank's buffer. */
FMOE_API int fmoe_ep_publish(const int32_t* cum, const uint64_t* peer_base, const fmoe_ep_layout_c* lay,
                             int32_t me, int32_t G, void* stream);
/* All ranks meet: each writes the barrier's epoch into every peer's flag word and waits, for
 * a bounded time (timeout_ms, 0 = about four seconds), until all peers wrote theirs; on expiry
 * the status word receives 0x300 | rank-not-seen and the kernel returns, so a missing rank never
 * hangs the GPU.  The epoch must grow by one per barrier on every rank: either pass it from
 * the host (`epoch`, epoch_counter = NULL) or let the kernel advance a device-side counter
 * (`epoch_counter`, one int32 per rank, zero-initialised), which keeps the launch identical
 * from step to step so a step can be captured in a CUDA graph. */
FMOE_API int fmoe_ep_barrier(const uint64_t* peer_base, const fmoe_ep_layout_c* lay, int32_t me,
                             int32_t G, int32_t epoch, int32_t* epoch_counter, int32_t* status,
                             int32_t timeout_ms, void* stream);
/* Sends every routed token row, with its local expert id, weight and return address, into
 * the owner rank's receive arrays; stores this rank's own received-row count in n_recv_dev.
 * Needs the count matrix complete (publish + barrier). */
FMOE_API int fmoe_ep_dispatch(const void* x, const int32_t* topk_ids, const float* topk_weight,
                              int32_t T, int32_t K, int32_t H, int32_t experts_per_rank,
                              const int32_t* order, const int32_t* cum, const uint64_t* peer_base,
                              const fmoe_ep_layout_c* lay, int32_t me, int32_t G, int32_t* n_recv_dev,
                              void* stream);
/* Sends the expert outputs of the received rows back to the send slot they came from. */
FMOE_API int fmoe_ep_return(const void* out_rows, int32_t H, const int32_t* n_recv_dev,
                            const uint64_t* peer_base, const fmoe_ep_layout_c* lay, int32_t me,
                            int32_t G, void* stream);

/* ---- Fused expert-parallel step (one process per GPU, at most 16 ranks): three kernels around the
 * local operator instead of eight.  All three read the step's epoch from the device word
 * `epoch_dev` (initialise it to 1); fmoe_ep_wait_combine advances it when the step is over, so the
 * launch arguments never change and a step can be captured in a CUDA graph.  Every wait is
 * bounded (timeout_ms, 0 = about four seconds): on expiry `status` receives 0x300 | rank-not-seen
 * (0x310 for the kernel's own grid barrier) and the kernel carries on without hanging the GPU.
 *
 * fmoe_ep_send: buckets this rank's T*K routed pairs by owner rank (stable), publishes the counts
 * to every rank, waits for everybody's counts, stores each token row with its local expert id,
 * weight and return address (source rank, pair index) into the owner's receive arrays, writes this
 * rank's received-row count to n_recv_dev and finally tells every rank that its rows are complete.
 * The kernel's CTAs meet at a barrier of their own: it must run with the GPU otherwise idle (it is
 * launched without programmatic overlap, after everything earlier on the stream).
 * scratch: int32[fmoe_ep_send_scratch_words(T, K, G)], zero-initialised once; the same array is
 * passed to all three kernels of the step (it also holds the words through which the CTAs of a
 * kernel share the outcome of a wait, so that only two of them poll memory the peers write). */
FMOE_API int64_t fmoe_ep_send_scratch_words(int32_t T, int32_t K, int32_t G);
FMOE_API int fmoe_ep_send(const void* x, const int32_t* topk_ids, const float* topk_weight, int32_t T, int32_t K,
                          int32_t H, int32_t experts_per_rank, const uint64_t* peer_base,
                          const fmoe_ep_layout_c* lay, int32_t me, int32_t G, int32_t* scratch,
                          const int32_t* epoch_dev, int32_t* n_recv_dev, int32_t* status, int32_t timeout_ms,
                          void* stream);
/* The same step with the token rows in any fixed-size encoding: row_bytes per row (a multiple of
 * 16), stored at lay->rows + slot * row_bytes on the owner, plus optional per-row scales
 * (scale_row_bytes, a multiple of 4, stored at lay->row_scales + slot * scale_row_bytes).  With rows
 * and scales from fmoe_quantise_rows the dispatch moves e4m3 instead of bf16 (half the bytes) and
 * the owner passes them to the operator as x / x_scale; results are bit-identical to sending bf16.
 * fmoe_ep_send(x, ..., H, ...) is this call with row_bytes = 2 * H and no scales. */
FMOE_API int fmoe_ep_send_rows(const void* rows, int32_t row_bytes, const void* row_scales, int32_t scale_row_bytes,
                               const int32_t* topk_ids, const float* topk_weight, int32_t T, int32_t K,
                               int32_t experts_per_rank, const uint64_t* peer_base, const fmoe_ep_layout_c* lay,
                               int32_t me, int32_t G, int32_t* scratch, const int32_t* epoch_dev,
                               int32_t* n_recv_dev, int32_t* status, int32_t timeout_ms, void* stream);
/* Waits until every rank's rows have arrived and fills row_ptrs[i] (i < *n_recv_dev) with the
 * address, in the source rank's `back` array, where the result of received row i belongs: the
 * partial_row_ptrs of the local fmoe_run. */
/* De-duplicated form of the fused step: one row per (token, owner rank) instead of per (token,
 * expert).  The owner receives the token's K-wide lists: ids [recv_cap, K] (local expert id, -1
 * where the expert lives on another rank), weights [recv_cap, K], src int32 [recv_cap, K] (routed
 * pair index on the source rank, -1 likewise) and src_rank [recv_cap]; n_recv_dev counts rows.
 * The owner runs the operator with K experts per row and fmoe_ep_recv_ready_dedup's row_ptrs
 * [recv_cap * K] as partial_row_ptrs; fmoe_ep_wait_combine is unchanged.  At most 256 tokens per
 * SM and rank.  Results are bit-identical to the form with one row per pair. */
FMOE_API int fmoe_ep_send_rows_dedup(const void* rows, int32_t row_bytes, const void* row_scales,
                                     int32_t scale_row_bytes, const int32_t* topk_ids, const float* topk_weight,
                                     int32_t T, int32_t K, int32_t experts_per_rank, const uint64_t* peer_base,
                                     const fmoe_ep_layout_c* lay, int32_t me, int32_t G, int32_t* scratch,
                                     const int32_t* epoch_dev, int32_t* n_recv_dev, int32_t* status,
                                     int32_t timeout_ms, void* stream);
FMOE_API int fmoe_ep_recv_ready_dedup(int32_t H, int32_t K, const int32_t* n_recv_dev, const uint64_t* peer_base,
                                      const fmoe_ep_layout_c* lay, int32_t me, int32_t G, const int32_t* epoch_dev,
                                      uint64_t* row_ptrs, int32_t* scratch, int32_t* status, int32_t timeout_ms,
                                      void* stream);
FMOE_API int fmoe_ep_recv_ready(int32_t H, const int32_t* n_recv_dev, const uint64_t* peer_base,
                                const fmoe_ep_layout_c* lay, int32_t me, int32_t G, const int32_t* epoch_dev,
                                uint64_t* row_ptrs, int32_t* scratch, int32_t* status, int32_t timeout_ms,
                                void* stream);
/* Waits until every rank has returned this rank's rows (the done_flag_* signal of their local
 * fmoe_run, aimed at flags_return) and adds them up: out[t] = bf16(sum over k ascending of
 * back[t*K + k]) in f32, pairs with an expert id outside [0, num_experts) skipped.  Advances the
 * epoch.  scratch: the step's scratch array (see fmoe_ep_send). */
FMOE_API int fmoe_ep_wait_combine(const int32_t* topk_ids, int32_t T, int32_t K, int32_t H, int32_t num_experts,
                                  const uint64_t* peer_base, const fmoe_ep_layout_c* lay, int32_t me, int32_t G,
                                  int32_t* epoch_dev, int32_t* scratch, void* out, int32_t* status,
                                  int32_t timeout_ms, void* stream);

/* What one fmoe_run with these traits and dimensions will launch on the current device: the
 * kernel flavour of each GEMM (the same decision fmoe_run takes) and the number of kernels
 * (moe_sorting is one launch below 8192 routed pairs and three from there on).  Only the
 * dimensions of `args` are read.  No counterpart in ck_tile. */
typedef struct fmoe_run_info_c {
  int32_t gemm1_kernel;   /* fmoe_gemm_kernel */
  int32_t gemm2_kernel;   /* fmoe_gemm_kernel */
  int32_t sort_launches;  /* 1 or 3 */
  int32_t quant_y_launch; /* 1 when the intermediate is quantised by a kernel of its own */
  int32_t launches;       /* kernels per fmoe_run */
  int32_t reserved[3];
} fmoe_run_info_c;
FMOE_API int fmoe_describe_run(const fmoe_traits_c* traits, const fmoe_args_c* args, fmoe_run_info_c* info);
/* Name of a kernel flavour ("fmoe_grouped_gemm_pair_kernel", ...), or "" for an unknown code. */
FMOE_API const char* fmoe_gemm_kernel_name(int32_t kernel);

#ifdef __cplusplus
} /* extern "C" */
#endif
#endif /* FMOE_B200_FUSED_MOE_C_H_ */
