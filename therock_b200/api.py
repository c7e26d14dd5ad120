"""ctypes binding of the C-ABI plus the Python mirror of the ck_tile host surface:
FusedMoeTraits / FusedMoeArgs / fused_moe(traits, args, stream) and moe_sorting."""
from __future__ import annotations

import ctypes
import os
from dataclasses import dataclass
from typing import Optional

import torch

# FMOE_B200_LIBRARY selects another build of the library (the bounds-checked or the timing-switch
# variant made by therock_b200.build); the default is the product library next to this file.
LIB_PATH = os.environ.get("FMOE_B200_LIBRARY") or os.path.join(os.path.dirname(os.path.abspath(__file__)),
                                                               "libfmoe_b200.so")

QUANT = {"none": 0, "token_channel": 1, "block128": 2, "block128_ue8m0": 3}
PARTIAL = {"f32": 0, "bf16": 1}


class FmoeError(RuntimeError):
    def __init__(self, code: int, msg: str):
        super().__init__(f"fmoe error {code}: {msg}")
        self.code = code


class _Traits(ctypes.Structure):
    _fields_ = [("quant", ctypes.c_int32), ("weight_dtype", ctypes.c_int32),
                ("activation", ctypes.c_int32), ("gate_only", ctypes.c_int32),
                ("block_m", ctypes.c_int32), ("gemm_mode", ctypes.c_int32), ("weight_layout", ctypes.c_int32),
                ("partial_dtype", ctypes.c_int32)]


class _RunInfo(ctypes.Structure):
    _fields_ = [("gemm1_kernel", ctypes.c_int32), ("gemm2_kernel", ctypes.c_int32),
                ("sort_launches", ctypes.c_int32), ("quant_y_launch", ctypes.c_int32),
                ("launches", ctypes.c_int32), ("reserved", ctypes.c_int32 * 3)]


class _Args(ctypes.Structure):
    _fields_ = [("x", ctypes.c_void_p), ("w1", ctypes.c_void_p), ("w2", ctypes.c_void_p),
                ("w1_scale", ctypes.c_void_p), ("w2_scale", ctypes.c_void_p),
                ("topk_ids", ctypes.c_void_p), ("topk_weight", ctypes.c_void_p),
                ("out", ctypes.c_void_p), ("workspace", ctypes.c_void_p),
                ("workspace_bytes", ctypes.c_uint64),
                ("T", ctypes.c_int32), ("H", ctypes.c_int32), ("I", ctypes.c_int32),
                ("E", ctypes.c_int32), ("K", ctypes.c_int32), ("expected_tokens", ctypes.c_int32),
                ("reserved", ctypes.c_int32 * 2), ("num_tokens_dev", ctypes.c_void_p),
                ("partial_row_ptrs", ctypes.c_void_p), ("done_flag_addrs", ctypes.c_void_p),
                ("done_flag_value", ctypes.c_void_p), ("done_counter", ctypes.c_void_p),
                ("done_flag_count", ctypes.c_int32), ("reserved2", ctypes.c_int32), ("x_scale", ctypes.c_void_p)]


class _Layout(ctypes.Structure):
    _fields_ = [("capacity", ctypes.c_int64)] + [(n, ctypes.c_uint64) for n in (
        "total_bytes", "meta", "sorted_token_ids", "sorted_weights", "sorted_rows",
        "sorted_expert_ids", "mblk_cum", "a_sorted", "a_scale", "y", "y_quant", "y_scale", "slots",
        "sort_scratch", "x_quant", "x_quant_scale")]


class EpLayout(ctypes.Structure):
    """Byte offsets inside the per-rank peer-addressable buffer (fmoe_ep_layout_c)."""
    _fields_ = [(n, ctypes.c_uint64) for n in ("flags", "matrix", "rows", "ids", "weights", "src", "back")] + \
               [("recv_cap", ctypes.c_int64), ("send_cap", ctypes.c_int64),
                ("flags_dispatch", ctypes.c_uint64), ("flags_return", ctypes.c_uint64), ("row_scales", ctypes.c_uint64),
                ("src_rank", ctypes.c_uint64)]


_lib: Optional[ctypes.CDLL] = None


def lib() -> ctypes.CDLL:
    """Loads libfmoe_b200.so; raises if it has not been built (there is no fallback)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise FmoeError(-100, f"{LIB_PATH} is missing: build it with "
                                  "`python -m therock_b200.build` (nvcc, sm_100a)")
        l = ctypes.CDLL(LIB_PATH)
        l.fmoe_version.restype = ctypes.c_int
        l.fmoe_last_error.restype = ctypes.c_char_p
        l.fmoe_sort_capacity.restype = ctypes.c_int64
        l.fmoe_sort_capacity.argtypes = [ctypes.c_int32] * 4
        l.fmoe_sort.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int32, ctypes.c_int32,
                                ctypes.c_int32, ctypes.c_int32, ctypes.c_void_p, ctypes.c_void_p,
                                ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p]
        l.fmoe_get_workspace_layout.argtypes = [ctypes.POINTER(_Traits), ctypes.POINTER(_Args),
                                                ctypes.POINTER(_Layout)]
        l.fmoe_get_workspace_size.argtypes = [ctypes.POINTER(_Traits), ctypes.POINTER(_Args),
                                              ctypes.POINTER(ctypes.c_uint64)]
        l.fmoe_run.argtypes = [ctypes.POINTER(_Traits), ctypes.POINTER(_Args), ctypes.c_void_p,
                               ctypes.POINTER(ctypes.c_float)]
        l.fmoe_run_static_ws.argtypes = [ctypes.POINTER(_Traits), ctypes.POINTER(_Args), ctypes.c_void_p]
        l.fmoe_check_status.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.POINTER(ctypes.c_int32)]
        l.fmoe_describe_run.argtypes = [ctypes.POINTER(_Traits), ctypes.POINTER(_Args), ctypes.POINTER(_RunInfo)]
        l.fmoe_gemm_kernel_name.argtypes = [ctypes.c_int32]
        l.fmoe_gemm_kernel_name.restype = ctypes.c_char_p
        l.fmoe_profile_create.argtypes = [ctypes.c_int32, ctypes.POINTER(ctypes.c_void_p)]
        l.fmoe_run_profiled.argtypes = [ctypes.POINTER(_Traits), ctypes.POINTER(_Args), ctypes.c_void_p,
                                        ctypes.c_void_p]
        l.fmoe_profile_read.argtypes = [ctypes.c_void_p, ctypes.POINTER(ctypes.c_float),
                                        ctypes.POINTER(ctypes.c_int32)]
        l.fmoe_profile_destroy.argtypes = [ctypes.c_void_p]
        l.fmoe_gather_rows.argtypes = [ctypes.c_void_p, ctypes.c_int32, ctypes.c_int32, ctypes.c_void_p,
                                       ctypes.c_int32, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p]
        l.fmoe_combine_rows.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int32, ctypes.c_int32,
                                        ctypes.c_int32, ctypes.c_void_p, ctypes.c_void_p]
        vp, i32 = ctypes.c_void_p, ctypes.c_int32
        l.fmoe_route.argtypes = [vp, i32, i32, i32, i32, vp, vp, vp]
        l.fmoe_ep_plan.argtypes = [vp, i32, i32, i32, i32, vp, vp, vp, vp, vp]
        l.fmoe_ep_publish.argtypes = [vp, vp, ctypes.POINTER(EpLayout), i32, i32, vp]
        l.fmoe_ep_barrier.argtypes = [vp, ctypes.POINTER(EpLayout), i32, i32, i32, vp, vp, i32, vp]
        l.fmoe_ep_dispatch.argtypes = [vp, vp, vp, i32, i32, i32, i32, vp, vp, vp, ctypes.POINTER(EpLayout),
                                       i32, i32, vp, vp]
        l.fmoe_ep_return.argtypes = [vp, i32, vp, vp, ctypes.POINTER(EpLayout), i32, i32, vp]
        l.fmoe_ep_send_scratch_words.restype = ctypes.c_int64
        l.fmoe_ep_send_scratch_words.argtypes = [i32, i32, i32]
        l.fmoe_ep_send.argtypes = [vp, vp, vp, i32, i32, i32, i32, vp, ctypes.POINTER(EpLayout), i32, i32, vp, vp,
                                   vp, vp, i32, vp]
        l.fmoe_ep_send_rows.argtypes = [vp, i32, vp, i32, vp, vp, i32, i32, i32, vp, ctypes.POINTER(EpLayout), i32, i32,
                                        vp, vp, vp, vp, i32, vp]
        l.fmoe_ep_send_rows_dedup.argtypes = l.fmoe_ep_send_rows.argtypes
        l.fmoe_ep_recv_ready_dedup.argtypes = [i32, i32, vp, vp, ctypes.POINTER(EpLayout), i32, i32, vp, vp, vp, vp, i32, vp]
        l.fmoe_quantise_rows.argtypes = [vp, i32, i32, i32, vp, vp, vp]
        l.fmoe_ep_recv_ready.argtypes = [i32, vp, vp, ctypes.POINTER(EpLayout), i32, i32, vp, vp, vp, vp, i32, vp]
        l.fmoe_ep_wait_combine.argtypes = [vp, i32, i32, i32, i32, vp, ctypes.POINTER(EpLayout), i32, i32, vp, vp, vp,
                                           vp, i32, vp]
        _lib = l
    return _lib


def _check(rc: int) -> None:
    if rc != 0:
        raise FmoeError(rc, lib().fmoe_last_error().decode())


@dataclass
class FusedMoeTraits:
    """Variant selection (role of ck_tile's fused_moe_traits)."""
    prec_i: str = "bf16"
    prec_w: str = "bf16"          # "bf16" | "fp8"
    prec_o: str = "bf16"
    quant: str = "none"           # "none" | "token_channel" | "block128" | "block128_ue8m0"
    activation: str = "silu"
    gate_only: int = 0
    block_m: int = 128
    gemm_mode: int = 0            # 0 = per-GEMM choice, 1 = single-CTA kernel, 2 = CTA-pair kernel
    weight_layout: str = "row_major"   # or "tiled128" (see therock_b200.weights.tile_weights)
    partial_dtype: str = "f32"    # "f32" | "bf16": how the K weighted expert outputs are held before the ordered sum

    def to_c(self) -> _Traits:
        if self.prec_i != "bf16" or self.prec_o != "bf16":
            raise FmoeError(-2, "activations and output are bf16")
        if self.quant not in QUANT:
            raise FmoeError(-1, f"unknown quant mode {self.quant!r}")
        if self.prec_w not in ("bf16", "fp8"):
            raise FmoeError(-1, f"unknown weight precision {self.prec_w!r}")
        if self.activation != "silu":
            raise FmoeError(-2, "only SiLU activation is built")
        t = _Traits()
        t.quant = QUANT[self.quant]
        t.weight_dtype = 0 if self.prec_w == "bf16" else 1
        t.activation = 0
        t.gate_only = self.gate_only
        t.block_m = self.block_m
        t.gemm_mode = self.gemm_mode
        if self.weight_layout not in ("row_major", "tiled128"):
            raise FmoeError(-1, f"unknown weight layout {self.weight_layout!r}")
        t.weight_layout = 0 if self.weight_layout == "row_major" else 1
        if self.partial_dtype not in PARTIAL:
            raise FmoeError(-1, f"unknown partial dtype {self.partial_dtype!r}")
        t.partial_dtype = PARTIAL[self.partial_dtype]
        return t


@dataclass
class FusedMoeArgs:
    """One call's tensors (role of ck_tile's fused_moe_args).  All CUDA tensors, contiguous."""
    a: torch.Tensor                       # [T, H] bf16
    g: torch.Tensor                       # [E, 2I, H] bf16 or float8_e4m3fn / uint8
    d: torch.Tensor                       # [E, H, I]
    topk_ids: torch.Tensor                # [T, K] int32
    topk_weight: torch.Tensor             # [T, K] float32
    o: Optional[torch.Tensor] = None      # [T, H] bf16 (allocated if None)
    g_scale: Optional[torch.Tensor] = None
    d_scale: Optional[torch.Tensor] = None
    workspace: Optional[torch.Tensor] = None   # uint8, >= fused_moe_workspace_size bytes
    num_tokens_dev: Optional[torch.Tensor] = None  # int32[1] on the device: process only that many tokens
    expected_tokens: int = 0                   # typical value of num_tokens_dev (kernel choice hint)
    partial_row_ptrs: Optional[torch.Tensor] = None  # int64 [T*K]: where each weighted partial row (bf16) goes
    done_flag_addrs: Optional[torch.Tensor] = None   # int64 [n]: addresses that receive done_flag_value[0] at the end
    done_flag_value: Optional[torch.Tensor] = None   # int32 [1] on the device
    done_counter: Optional[torch.Tensor] = None      # int32 [1] on the device, zero
    a_scale: Optional[torch.Tensor] = None           # scales of `a` when `a` already holds e4m3 rows (quantise_rows)

    def to_c(self, gate_only: bool = False) -> _Args:
        for name in ("a", "g", "d", "topk_ids", "topk_weight"):
            t = getattr(self, name)
            if not (t.is_cuda and t.is_contiguous()):
                raise FmoeError(-1, f"{name} must be a contiguous CUDA tensor")
        if self.a_scale is not None:
            if self.a.element_size() != 1:
                raise FmoeError(-1, "a must hold e4m3 bytes when a_scale is given")
        elif self.a.dtype != torch.bfloat16:
            raise FmoeError(-1, "a must be bf16")
        if self.topk_ids.dtype != torch.int32 or self.topk_weight.dtype != torch.float32:
            raise FmoeError(-1, "topk_ids must be int32 and topk_weight float32")
        T, H = self.a.shape
        E, I2, H2 = self.g.shape
        I = I2 if gate_only else I2 // 2
        if H2 != H or tuple(self.d.shape) != (E, H, I) or (not gate_only and I2 % 2):
            raise FmoeError(-1, "weight shapes do not match [E,2I,H] ([E,I,H] when gate_only) / [E,H,I]")
        if self.topk_ids.shape[0] != T or self.topk_weight.shape != self.topk_ids.shape:
            raise FmoeError(-1, "topk tensors must be [T, K]")
        c = _Args()
        c.x, c.w1, c.w2 = self.a.data_ptr(), self.g.data_ptr(), self.d.data_ptr()
        c.w1_scale = self.g_scale.data_ptr() if self.g_scale is not None else None
        c.w2_scale = self.d_scale.data_ptr() if self.d_scale is not None else None
        c.topk_ids, c.topk_weight = self.topk_ids.data_ptr(), self.topk_weight.data_ptr()
        c.out = self.o.data_ptr() if self.o is not None else None
        if self.workspace is not None:
            c.workspace = self.workspace.data_ptr()
            c.workspace_bytes = self.workspace.numel() * self.workspace.element_size()
        c.T, c.H, c.I, c.E, c.K = T, H, I, E, self.topk_ids.shape[1]
        c.num_tokens_dev = self.num_tokens_dev.data_ptr() if self.num_tokens_dev is not None else None
        c.expected_tokens = int(self.expected_tokens)
        if self.a_scale is not None:
            c.x_scale = self.a_scale.data_ptr()
        if self.partial_row_ptrs is not None:
            c.partial_row_ptrs = self.partial_row_ptrs.data_ptr()
        if self.done_flag_addrs is not None:
            c.done_flag_addrs = self.done_flag_addrs.data_ptr()
            c.done_flag_count = self.done_flag_addrs.numel()
            c.done_flag_value = self.done_flag_value.data_ptr()
            c.done_counter = self.done_counter.data_ptr()
        return c


def sort_capacity(T: int, K: int, E: int, block_m: int = 128) -> int:
    return int(lib().fmoe_sort_capacity(T, K, E, block_m))


def describe_run(traits: FusedMoeTraits, args: FusedMoeArgs) -> dict:
    """What fmoe_run will launch for these traits and dimensions on the current device: the
    kernel flavour of each GEMM (name as compiled) and the number of kernels per run."""
    t, a, info = traits.to_c(), args.to_c(bool(traits.gate_only)), _RunInfo()
    _check(lib().fmoe_describe_run(ctypes.byref(t), ctypes.byref(a), ctypes.byref(info)))
    d = {n: int(getattr(info, n)) for n, _ in _RunInfo._fields_ if n != "reserved"}
    d["gemm1_kernel_name"] = lib().fmoe_gemm_kernel_name(info.gemm1_kernel).decode()
    d["gemm2_kernel_name"] = lib().fmoe_gemm_kernel_name(info.gemm2_kernel).decode()
    return d


def launches_per_run(traits: FusedMoeTraits, args: FusedMoeArgs) -> int:
    return describe_run(traits, args)["launches"]


def workspace_layout(traits: FusedMoeTraits, args: FusedMoeArgs) -> dict:
    t, a, l = traits.to_c(), args.to_c(bool(traits.gate_only)), _Layout()
    _check(lib().fmoe_get_workspace_layout(ctypes.byref(t), ctypes.byref(a), ctypes.byref(l)))
    return {n: int(getattr(l, n)) for n, _ in _Layout._fields_}


def fused_moe_workspace_size(traits: FusedMoeTraits, args: FusedMoeArgs) -> int:
    t, a, n = traits.to_c(), args.to_c(bool(traits.gate_only)), ctypes.c_uint64(0)
    _check(lib().fmoe_get_workspace_size(ctypes.byref(t), ctypes.byref(a), ctypes.byref(n)))
    return int(n.value)


def _stream_ptr(stream) -> int:
    if stream is None:
        stream = torch.cuda.current_stream()
    return int(stream.cuda_stream) if hasattr(stream, "cuda_stream") else int(stream)


def fused_moe(traits: FusedMoeTraits, args: FusedMoeArgs, stream=None, time_kernel: bool = False):
    """Enqueues the fused operator on `stream` (torch current stream by default).
    Returns the output tensor, or (output, elapsed_ms) when time_kernel is set.  Missing
    output / workspace tensors are allocated here with torch (callers on a hot loop pass
    their own)."""
    if args.o is None:
        args.o = torch.empty(args.a.shape, dtype=torch.bfloat16, device=args.a.device)
    if args.workspace is None:
        args.workspace = torch.empty(fused_moe_workspace_size(traits, args), dtype=torch.uint8,
                                     device=args.a.device)
    t, a = traits.to_c(), args.to_c(bool(traits.gate_only))
    ms = ctypes.c_float(0.0)
    _check(lib().fmoe_run(ctypes.byref(t), ctypes.byref(a), _stream_ptr(stream),
                          ctypes.byref(ms) if time_kernel else None))
    return (args.o, float(ms.value)) if time_kernel else args.o


def check_status(workspace: torch.Tensor, stream=None) -> int:
    st = ctypes.c_int32(0)
    _check(lib().fmoe_check_status(workspace.data_ptr(), _stream_ptr(stream), ctypes.byref(st)))
    return int(st.value)


def moe_sorting(topk_ids: torch.Tensor, topk_weight: torch.Tensor, num_experts: int,
                block_m: int = 128, stream=None):
    """Returns (sorted_token_ids, sorted_weights, sorted_expert_ids, num_tokens_post_pad)."""
    if not (topk_ids.is_cuda and topk_ids.dtype == torch.int32 and topk_ids.is_contiguous()):
        raise FmoeError(-1, "topk_ids must be a contiguous CUDA int32 tensor")
    T, K = topk_ids.shape
    cap = sort_capacity(T, K, num_experts, block_m)
    dev = topk_ids.device
    ids = torch.empty(cap, dtype=torch.int32, device=dev)
    w = torch.empty(cap, dtype=torch.float32, device=dev)
    eids = torch.empty(cap // block_m, dtype=torch.int32, device=dev)
    npp = torch.empty(1, dtype=torch.int32, device=dev)
    _check(lib().fmoe_sort(topk_ids.data_ptr(), topk_weight.data_ptr(), T, K, num_experts, block_m,
                           ids.data_ptr(), w.data_ptr(), eids.data_ptr(), npp.data_ptr(),
                           _stream_ptr(stream)))
    return ids, w, eids, npp


STAGES = ("sort", "gather", "gemm1", "quant_y", "gemm2", "combine")


class StageProfile:
    """Per-kernel timing of fused_moe runs: events are recorded between the kernels and read
    after the timed loop, so nothing synchronises inside it."""

    def __init__(self, max_runs: int):
        self._h = ctypes.c_void_p()
        _check(lib().fmoe_profile_create(max_runs, ctypes.byref(self._h)))

    def run(self, traits: FusedMoeTraits, args: FusedMoeArgs, stream=None):
        t, a = traits.to_c(), args.to_c(bool(traits.gate_only))
        _check(lib().fmoe_run_profiled(ctypes.byref(t), ctypes.byref(a), _stream_ptr(stream), self._h))
        return args.o

    def read(self) -> dict:
        """Waits for the recorded runs; returns {'runs': n, stage: total_ms, ...}."""
        ms = (ctypes.c_float * 6)()
        n = ctypes.c_int32(0)
        _check(lib().fmoe_profile_read(self._h, ms, ctypes.byref(n)))
        d = {name: float(ms[i]) for i, name in enumerate(STAGES)}
        d["runs"] = int(n.value)
        return d

    def close(self):
        if self._h:
            lib().fmoe_profile_destroy(self._h)
            self._h = ctypes.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def gather_rows(src: torch.Tensor, row_ids: torch.Tensor, n_rows_dev: torch.Tensor,
                out: Optional[torch.Tensor] = None, stream=None) -> torch.Tensor:
    """out[i] = src[row_ids[i]] for i < n_rows_dev[0] (bf16 rows; ids outside the source give
    zero rows).  The expert-parallel dispatch uses it to pack rows per destination rank."""
    n = row_ids.numel()
    if out is None:
        out = torch.empty(n, src.shape[1], dtype=src.dtype, device=src.device)
    _check(lib().fmoe_gather_rows(src.data_ptr(), src.shape[0], src.shape[1], row_ids.data_ptr(), n,
                                  n_rows_dev.data_ptr(), out.data_ptr(), _stream_ptr(stream)))
    return out


def quant_scale_row_bytes(quant: str, hidden: int) -> int:
    """Bytes of one row of activation scales in the given fp8 quant mode."""
    if quant == "token_channel":
        return 4
    if quant == "block128":
        return 4 * (hidden // 128)
    if quant == "block128_ue8m0":
        return (hidden // 128 + 3) // 4 * 4
    raise FmoeError(-1, f"{quant!r} is not an fp8 quant mode")


def quantise_rows(x: torch.Tensor, quant: str, q: Optional[torch.Tensor] = None,
                  scales: Optional[torch.Tensor] = None, stream=None):
    """The operator's dynamic e4m3 quantisation of activation rows as a call of its own.
    Returns (q uint8 [T, H], scales uint8 [T, quant_scale_row_bytes]); pass them as
    FusedMoeArgs.a / a_scale and the operator's result is bit-identical to passing x."""
    T, H = x.shape
    if q is None:
        q = torch.empty(T, H, dtype=torch.uint8, device=x.device)
    if scales is None:
        scales = torch.empty(T, quant_scale_row_bytes(quant, H), dtype=torch.uint8, device=x.device)
    _check(lib().fmoe_quantise_rows(x.data_ptr(), T, H, QUANT[quant], q.data_ptr(), scales.data_ptr(),
                                    _stream_ptr(stream)))
    return q, scales


def combine_rows(rows: torch.Tensor, index: torch.Tensor, T: int, K: int,
                 out: Optional[torch.Tensor] = None, stream=None) -> torch.Tensor:
    """out[t] = bf16(sum_k rows[index[t*K+k]]), k ascending, f32 accumulation, index < 0 skipped."""
    H = rows.shape[1]
    if out is None:
        out = torch.empty(T, H, dtype=torch.bfloat16, device=rows.device)
    _check(lib().fmoe_combine_rows(rows.data_ptr(), index.data_ptr(), T, K, H, out.data_ptr(),
                                   _stream_ptr(stream)))
    return out


STATIC_WS_BYTES = 64 * 1024 * 1024


def fused_moe_static_ws(traits: FusedMoeTraits, args: FusedMoeArgs, stream=None) -> torch.Tensor:
    """fused_moe for hosts that may not allocate device memory: the scratch comes from the
    64 MiB array built into the library (fmoe_run_static_ws).  The caller passes inputs and
    the output tensor; nothing is allocated here either, so args.o is required.  Calls on
    one device share that array: keep them on one stream."""
    if args.o is None:
        raise FmoeError(-1, "the output tensor must be provided (this entry point allocates nothing)")
    t, a = traits.to_c(), args.to_c(bool(traits.gate_only))
    _check(lib().fmoe_run_static_ws(ctypes.byref(t), ctypes.byref(a), _stream_ptr(stream)))
    return args.o


class HostPipeline:
    """Runs an operator step on host-resident batches with the copies hidden behind compute.

    Three streams: host->device copies of batch i+1 and the device->host copy of result i-1
    overlap the compute of batch i (`depth` device-side input/output slots).  Every batch is
    still copied in from pinned host memory and its result copied back; only the waiting is
    removed.  `step(x, topk_ids, topk_weight, slot) -> out` runs on the compute stream; `slot`
    (0..depth-1) lets the step keep one preallocated output per slot."""

    def __init__(self, step, T: int, H: int, K: int, device, depth: int = 2):
        self.step, self.depth, self.device = step, depth, device
        self.h2d, self.compute, self.d2h = (torch.cuda.Stream(device) for _ in range(3))
        self.x = [torch.empty(T, H, dtype=torch.bfloat16, device=device) for _ in range(depth)]
        self.ids = [torch.empty(T, K, dtype=torch.int32, device=device) for _ in range(depth)]
        self.w = [torch.empty(T, K, dtype=torch.float32, device=device) for _ in range(depth)]
        self.out = [None] * depth
        self.in_ready = [torch.cuda.Event() for _ in range(depth)]
        self.in_free = [torch.cuda.Event() for _ in range(depth)]
        self.out_ready = [torch.cuda.Event() for _ in range(depth)]
        self.out_free = [torch.cuda.Event() for _ in range(depth)]
        self.n = 0

    def submit(self, x_host, ids_host, w_host, out_host):
        s = self.n % self.depth
        first = self.n < self.depth
        with torch.cuda.stream(self.h2d):
            if not first:
                self.h2d.wait_event(self.in_free[s])        # the compute that read this slot is done
            self.x[s].copy_(x_host, non_blocking=True)
            self.ids[s].copy_(ids_host, non_blocking=True)
            self.w[s].copy_(w_host, non_blocking=True)
            self.in_ready[s].record(self.h2d)
        with torch.cuda.stream(self.compute):
            self.compute.wait_event(self.in_ready[s])
            if not first:
                self.compute.wait_event(self.out_free[s])   # the previous result of this slot left
            out = self.step(self.x[s], self.ids[s], self.w[s], s)
            self.out[s] = out
            self.in_free[s].record(self.compute)
            self.out_ready[s].record(self.compute)
        with torch.cuda.stream(self.d2h):
            self.d2h.wait_event(self.out_ready[s])
            out_host.copy_(out, non_blocking=True)
            self.out_free[s].record(self.d2h)
        self.n += 1

    def mark(self) -> "torch.cuda.Event":
        """Event on the compute stream that follows everything submitted so far on all three
        streams (for timing a batch of submissions on the device)."""
        ev_a, ev_b = torch.cuda.Event(), torch.cuda.Event()
        ev_a.record(self.h2d)
        ev_b.record(self.d2h)
        self.compute.wait_event(ev_a)
        self.compute.wait_event(ev_b)
        ev = torch.cuda.Event(enable_timing=True)
        ev.record(self.compute)
        return ev

    def drain(self):
        self.d2h.synchronize()
        self.compute.synchronize()
        self.h2d.synchronize()


def append_shared_expert(topk_ids: torch.Tensor, topk_weight: torch.Tensor, shared_expert_id: int,
                         weight: float = 1.0):
    """A shared expert (a dense FFN every token passes through, added to the routed experts'
    output, as in DeepSeek-style layers) fused into the same operator call: store its weights as
    expert `shared_expert_id` of W1 / W2 and give every token one more (expert, weight) pair.  The
    shared expert's rows then run through the same grouped GEMMs as one large group and its
    output is added in the same ordered combine (it is the last term of every token's sum).
    Returns (topk_ids [T, K+1], topk_weight [T, K+1])."""
    T = topk_ids.shape[0]
    ids = torch.cat([topk_ids, torch.full((T, 1), shared_expert_id, dtype=topk_ids.dtype, device=topk_ids.device)], dim=1)
    w = torch.cat([topk_weight, torch.full((T, 1), weight, dtype=topk_weight.dtype, device=topk_weight.device)], dim=1)
    return ids.contiguous(), w.contiguous()


def route(logits: torch.Tensor, topk: int, mode: str = "softmax", stream=None):
    """Router kernel: logits [T, E] f32 (CUDA) -> (topk_ids int32 [T, K], topk_weight f32 [T, K])."""
    if not (logits.is_cuda and logits.dtype == torch.float32 and logits.is_contiguous()):
        raise FmoeError(-1, "logits must be a contiguous CUDA float32 tensor")
    T, E = logits.shape
    ids = torch.empty(T, topk, dtype=torch.int32, device=logits.device)
    w = torch.empty(T, topk, dtype=torch.float32, device=logits.device)
    _check(lib().fmoe_route(logits.data_ptr(), T, E, topk, 0 if mode == "softmax" else 1, ids.data_ptr(),
                            w.data_ptr(), _stream_ptr(stream)))
    return ids, w


class GraphPipeline:
    """Host-resident batches with one CUDA-graph launch per step.

    Two device-side slots.  The graph of slot s holds three independent branches that run
    concurrently on the device: the operator step on slot s (whose inputs the previous replay
    copied in), the host->device copy of the next batch into slot s^1, and the device->host copy of
    the result the previous replay computed in slot s^1.  Consecutive replays alternate between
    the two graphs, so every step still moves its inputs in from pinned host memory and its result
    back out, the copies hide behind the neighbouring step's compute, and the host issues a single
    launch per step (the Python-side stream and event calls of HostPipeline are gone from the loop).

    step(x, topk_ids, topk_weight, slot) -> output tensor; it must write a tensor that is fixed per
    slot (capture records addresses) and must neither allocate nor synchronise.
    The host buffers are fixed at construction: x_host [T, H] bf16, ids_host [T, K] int32,
    w_host [T, K] f32, out_host [T, H] bf16, all pinned.  The constructor copies the first batch
    in.  submit() number i (from 0) computes batch i, copies in whatever the host buffers hold while
    it runs (batch i+1: fill them before the call and leave them alone until it has completed) and
    copies the result of batch i-1 to out_host; flush() delivers the last result."""

    def __init__(self, step, x_host, ids_host, w_host, out_host, device):
        T, H = x_host.shape
        K = ids_host.shape[1]
        self.device = device
        self.main, self.s_in, self.s_out = (torch.cuda.Stream(device) for _ in range(3))
        self.x = [torch.empty(T, H, dtype=torch.bfloat16, device=device) for _ in range(2)]
        self.ids = [torch.empty(T, K, dtype=torch.int32, device=device) for _ in range(2)]
        self.w = [torch.empty(T, K, dtype=torch.float32, device=device) for _ in range(2)]
        self.hosts = (x_host, ids_host, w_host, out_host)
        self.n = 0
        with torch.cuda.stream(self.main):
            # warm-up outside capture (lazy initialisation, per-slot output tensors)
            self.out = []
            for s in range(2):
                self._copy_in(s)
                self.out.append(step(self.x[s], self.ids[s], self.w[s], s))
            self.main.synchronize()
            self.graphs = []
            for s in range(2):
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=self.main):
                    fork = torch.cuda.Event()
                    fork.record(self.main)
                    self.s_in.wait_event(fork)
                    self.s_out.wait_event(fork)
                    with torch.cuda.stream(self.s_in):
                        self._copy_in(s ^ 1)
                        j_in = torch.cuda.Event()
                        j_in.record(self.s_in)
                    with torch.cuda.stream(self.s_out):
                        out_host.copy_(self.out[s ^ 1], non_blocking=True)
                        j_out = torch.cuda.Event()
                        j_out.record(self.s_out)
                    step(self.x[s], self.ids[s], self.w[s], s)
                    self.main.wait_event(j_in)
                    self.main.wait_event(j_out)
                self.graphs.append(g)
            self._copy_in(0)              # the first batch is in place before the first replay
            self.main.synchronize()

    def _copy_in(self, s):
        x_host, ids_host, w_host, _ = self.hosts
        self.x[s].copy_(x_host, non_blocking=True)
        self.ids[s].copy_(ids_host, non_blocking=True)
        self.w[s].copy_(w_host, non_blocking=True)

    def submit(self):
        """One step: a single graph launch on the pipeline's stream."""
        with torch.cuda.stream(self.main):
            self.graphs[self.n & 1].replay()
        self.n += 1

    def mark(self) -> "torch.cuda.Event":
        ev = torch.cuda.Event(enable_timing=True)
        ev.record(self.main)
        return ev

    def flush(self):
        """Copies the last computed result out and waits for everything."""
        with torch.cuda.stream(self.main):
            if self.n:
                self.hosts[3].copy_(self.out[(self.n - 1) & 1], non_blocking=True)
        self.main.synchronize()
