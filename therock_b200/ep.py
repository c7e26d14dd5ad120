"""Expert-parallel fused MoE: one process per GPU, experts sharded by contiguous ranges,
tokens data-parallel.  Each step is

    route (given) -> pack rows per destination rank (CUDA gather kernel)
    -> all-to-all dispatch (NCCL over NVLink, torch.distributed)
    -> local fused_moe on the received rows (each row is a one-expert token)
    -> all-to-all return -> ordered k-sum into the local output (CUDA combine kernel).

The reference operator is single-GPU; this wrapper is the partitioning the benchmark
configurations ask for (1 expert per GPU at 8 GPUs for the Mixtral shape).  The same code
runs on CPU tensors with the gloo backend for the host-side logic tests, with the two CUDA
kernels and the local operator replaced by callables the test injects.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Optional

import torch
import torch.distributed as dist


@dataclass
class DispatchPlan:
    """Host-side description of one dispatch (all tensors live on the compute device)."""
    order: torch.Tensor          # [R] flat pair index (t*K+k) of each send slot, grouped by dest rank
    send_counts: list            # rows sent to each rank
    recv_counts: list            # rows received from each rank
    inv_index: torch.Tensor      # [T*K] send slot of each pair, -1 if the pair is dropped
    n_send: int
    n_recv: int


def plan_dispatch(topk_ids: torch.Tensor, experts_per_rank: int, world: int, group=None,
                  timeout_s=None) -> DispatchPlan:
    """Stable grouping of the routed pairs by destination rank and the count exchange."""
    flat = topk_ids.reshape(-1).to(torch.int64)
    n_exp = experts_per_rank * world
    valid = (flat >= 0) & (flat < n_exp)
    dest = torch.where(valid, flat // experts_per_rank, torch.full_like(flat, world))
    order = torch.argsort(dest, stable=True)
    counts = torch.bincount(dest, minlength=world + 1)[:world]
    n_send = int(counts.sum().item())
    order = order[:n_send]
    send_counts_t = counts.to(torch.int64)
    recv_counts_t = torch.empty_like(send_counts_t)
    _a2a(recv_counts_t, send_counts_t, None, None, world, group, timeout_s, "count exchange")
    send_counts = send_counts_t.tolist()
    recv_counts = recv_counts_t.tolist()
    inv = torch.full((flat.numel(),), -1, dtype=torch.int32, device=flat.device)
    inv[order] = torch.arange(n_send, dtype=torch.int32, device=flat.device)
    return DispatchPlan(order=order, send_counts=send_counts, recv_counts=recv_counts, inv_index=inv,
                        n_send=n_send, n_recv=int(sum(recv_counts)))


@dataclass
class DedupPlan:
    """One send row per (token, destination rank) instead of one per (token, expert)."""
    tok: torch.Tensor            # [n_send] token of each send row, grouped by destination rank
    ids: torch.Tensor            # [n_send, K] expert ids local to the destination, -1 where the pair goes elsewhere
    weights: torch.Tensor        # [n_send, K] routing weights at the same positions (0 where unused)
    send_counts: list
    recv_counts: list
    index: torch.Tensor          # [T * world] send row of (token, rank), -1 if the token sends nothing there
    n_send: int
    n_recv: int


def plan_dispatch_dedup(topk_ids: torch.Tensor, topk_weight: torch.Tensor, experts_per_rank: int, world: int,
                        group=None, timeout_s=None) -> DedupPlan:
    """Groups a token's pairs by owning rank: a token whose K experts live on d distinct ranks
    sends d rows (each with the K-wide id/weight lists of that rank, k positions kept) instead of K."""
    T, K = topk_ids.shape
    dev = topk_ids.device
    ids = topk_ids.to(torch.int64)
    n_exp = experts_per_rank * world
    valid = (ids >= 0) & (ids < n_exp)
    dest = torch.where(valid, ids // experts_per_rank, torch.full_like(ids, world))          # [T, K]
    hit = torch.zeros(T, world + 1, dtype=torch.bool, device=dev)
    hit.scatter_(1, dest, True)
    hit = hit[:, :world]                                                                     # [T, world]
    # send rows ordered by (rank, token): column-major walk over `hit`
    rank_of, tok = torch.nonzero(hit.t(), as_tuple=True)
    n_send = int(tok.numel())
    counts = hit.sum(dim=0).to(torch.int64)
    index = torch.full((T * world,), -1, dtype=torch.int32, device=dev)
    index[tok * world + rank_of] = torch.arange(n_send, dtype=torch.int32, device=dev)
    mine = dest[tok] == rank_of.unsqueeze(1)                                                 # [n_send, K]
    row_ids = torch.where(mine, ids[tok] % experts_per_rank, torch.full_like(ids[tok], -1)).to(torch.int32)
    row_w = torch.where(mine, topk_weight[tok], torch.zeros_like(topk_weight[tok]))
    recv_counts_t = torch.empty_like(counts)
    _a2a(recv_counts_t, counts, None, None, world, group, timeout_s, "count exchange")
    recv_counts = recv_counts_t.tolist()
    return DedupPlan(tok=tok.to(torch.int32), ids=row_ids.contiguous(), weights=row_w.contiguous(),
                     send_counts=counts.tolist(), recv_counts=recv_counts, index=index, n_send=n_send,
                     n_recv=int(sum(recv_counts)))


class ExpertParallelTimeout(RuntimeError):
    """A collective of the expert-parallel step did not complete within its limit: a peer rank is
    missing or stuck.  The process group should be torn down; the step's buffers are undefined."""


def _wait(work, timeout_s, what):
    """Waits for an asynchronous collective with the step's own limit.  (With the NCCL backend
    torch's watchdog additionally polls the communicator's asynchronous error state and aborts it
    after the process group's timeout; this limit is usually much shorter.)"""
    import datetime
    try:
        ok = work.wait(timeout=datetime.timedelta(seconds=timeout_s))
    except RuntimeError as exc:           # gloo raises on expiry, NCCL returns or raises depending on the mode
        raise ExpertParallelTimeout(f"{what} did not complete within {timeout_s} s: {exc}") from exc
    if ok is False:
        raise ExpertParallelTimeout(f"{what} did not complete within {timeout_s} s")


def _a2a(out: torch.Tensor, inp: torch.Tensor, out_splits, in_splits, world: int, group=None, timeout_s=None,
         what="all-to-all"):
    if world > 1:
        if timeout_s is None:
            dist.all_to_all_single(out, inp, out_splits, in_splits, group=group)
        else:
            _wait(dist.all_to_all_single(out, inp, out_splits, in_splits, group=group, async_op=True), timeout_s, what)
    else:
        out.copy_(inp)


class ExpertParallelMoE:
    """Holds one rank's expert shard and runs dispatch -> local operator -> combine.

    local_moe(x_rows [n,H], expert_ids [n,1] int32 local ids, weights [n,1] f32) -> [n,H] bf16
    gather(src [T,H], row_ids [n] int32) -> [n,H];  combine(rows [n,H], index [T*K] int32, T, K) -> [T,H]
    default to the CUDA kernels of this library.
    """

    def __init__(self, num_experts: int, world: int, rank: int, local_moe: Callable,
                 gather: Optional[Callable] = None, combine: Optional[Callable] = None, group=None,
                 dedup: bool = False, timeout_s: Optional[float] = None):
        if num_experts % world:
            raise ValueError("experts must divide evenly over ranks")
        self.E, self.world, self.rank, self.group = num_experts, world, rank, group
        # dedup: one row per (token, destination rank); the owner sums the token's local experts
        # (k ascending) and returns one partial row, the sender adds the partials in rank order
        self.dedup = dedup
        # failure detection: with a limit every collective of the step is waited for on the host
        # and a missing peer raises ExpertParallelTimeout instead of blocking for the process
        # group's (much longer) timeout
        self.timeout_s = timeout_s
        self.e_local = num_experts // world
        self.local_moe = local_moe
        self.gather = gather or _cuda_gather
        self.combine = combine or _cuda_combine
        self.trace = None          # set to [] to collect (phase, cuda event) marks per forward

    def _mark(self, name):
        if self.trace is not None:
            ev = torch.cuda.Event(enable_timing=True)
            ev.record()
            self.trace.append((name, ev))

    def _forward_dedup(self, x: torch.Tensor, topk_ids: torch.Tensor, topk_weight: torch.Tensor) -> torch.Tensor:
        T, H = x.shape
        K = topk_ids.shape[1]
        dev = x.device
        self._mark("start")
        plan = plan_dispatch_dedup(topk_ids, topk_weight, self.e_local, self.world, self.group, self.timeout_s)
        self._mark("plan")
        send_rows = self.gather(x, plan.tok)
        send_meta = torch.cat([plan.ids.to(torch.float32), plan.weights.to(torch.float32)], dim=1).contiguous()
        self._mark("pack")
        recv_rows = torch.empty(plan.n_recv, H, dtype=x.dtype, device=dev)
        recv_meta = torch.empty(plan.n_recv, 2 * K, dtype=torch.float32, device=dev)
        _a2a(recv_rows, send_rows, plan.recv_counts, plan.send_counts, self.world, self.group, self.timeout_s)
        _a2a(recv_meta, send_meta, plan.recv_counts, plan.send_counts, self.world, self.group, self.timeout_s)
        self._mark("dispatch")
        ids_local = recv_meta[:, :K].to(torch.int32).contiguous()       # -1 entries are skipped by the operator
        w_local = recv_meta[:, K:].contiguous()
        part = self.local_moe(recv_rows, ids_local, w_local) if plan.n_recv > 0 else recv_rows
        self._mark("local_moe")
        back = torch.empty(plan.n_send, H, dtype=x.dtype, device=dev)
        _a2a(back, part, plan.send_counts, plan.recv_counts, self.world, self.group, self.timeout_s)
        self._mark("return")
        out = self.combine(back, plan.index, T, self.world)             # partial rows added in rank order
        self._mark("combine")
        return out

    def forward(self, x: torch.Tensor, topk_ids: torch.Tensor, topk_weight: torch.Tensor) -> torch.Tensor:
        if self.dedup:
            return self._forward_dedup(x, topk_ids, topk_weight)
        T, H = x.shape
        K = topk_ids.shape[1]
        self._mark("start")
        plan = plan_dispatch(topk_ids, self.e_local, self.world, self.group, self.timeout_s)
        self._mark("plan")
        dev = x.device
        order32 = plan.order.to(torch.int32)
        tok = torch.div(order32, K, rounding_mode="floor").to(torch.int32)
        # pack: rows, local expert id and weight of every send slot
        send_rows = self.gather(x, tok)
        flat_ids = topk_ids.reshape(-1)[plan.order]
        send_meta = torch.stack([(flat_ids % self.e_local).to(torch.float32),
                                 topk_weight.reshape(-1)[plan.order]], dim=1).contiguous()
        self._mark("pack")
        recv_rows = torch.empty(plan.n_recv, H, dtype=x.dtype, device=dev)
        recv_meta = torch.empty(plan.n_recv, 2, dtype=torch.float32, device=dev)
        _a2a(recv_rows, send_rows, plan.recv_counts, plan.send_counts, self.world, self.group, self.timeout_s)
        _a2a(recv_meta, send_meta, plan.recv_counts, plan.send_counts, self.world, self.group, self.timeout_s)
        self._mark("dispatch")
        # local experts: every received row is a token with a single expert
        ids_local = recv_meta[:, 0].to(torch.int32).reshape(-1, 1).contiguous()
        w_local = recv_meta[:, 1].reshape(-1, 1).contiguous()
        part = self.local_moe(recv_rows, ids_local, w_local) if plan.n_recv > 0 else recv_rows
        self._mark("local_moe")
        # return trip and ordered reduction
        back = torch.empty(plan.n_send, H, dtype=x.dtype, device=dev)
        _a2a(back, part, plan.send_counts, plan.recv_counts, self.world, self.group, self.timeout_s)
        self._mark("return")
        out = self.combine(back, plan.inv_index, T, K)
        self._mark("combine")
        return out


def _cuda_gather(src: torch.Tensor, row_ids: torch.Tensor) -> torch.Tensor:
    from . import api
    n = torch.tensor([row_ids.numel()], dtype=torch.int32, device=src.device)
    if row_ids.numel() == 0:
        return torch.empty(0, src.shape[1], dtype=src.dtype, device=src.device)
    return api.gather_rows(src, row_ids.contiguous(), n)


def _cuda_combine(rows: torch.Tensor, index: torch.Tensor, T: int, K: int) -> torch.Tensor:
    from . import api
    if rows.shape[0] == 0:
        rows = torch.zeros(1, rows.shape[1], dtype=rows.dtype, device=rows.device)
    return api.combine_rows(rows, index.contiguous(), T, K)


def make_local_moe(traits, w1_local, w2_local, w1_scale=None, w2_scale=None):
    """Local operator over this rank's expert shard using the CUDA library."""
    from . import api

    cache = {}

    def run(x_rows, ids_local, w_local):
        n = x_rows.shape[0]
        args = api.FusedMoeArgs(a=x_rows, g=w1_local, d=w2_local, topk_ids=ids_local, topk_weight=w_local,
                                g_scale=w1_scale, d_scale=w2_scale)
        need = api.fused_moe_workspace_size(traits, args)
        ws = cache.get("ws")
        if ws is None or ws.numel() < need:
            ws = torch.empty(need, dtype=torch.uint8, device=x_rows.device)
            cache["ws"] = ws
        args.workspace = ws
        args.o = torch.empty(n, x_rows.shape[1], dtype=torch.bfloat16, device=x_rows.device)
        return api.fused_moe(traits, args)

    return run


class PeerExpertParallelMoE:
    """Expert parallelism over NVLink peer memory with no host synchronisation.

    Every rank owns one peer-addressable buffer (torch symmetric memory, NVLS multicast not
    used).  A step is a fixed sequence of asynchronous launches on the current stream.

    fused=True (default, at most 16 ranks): seven launches --
        send (bucket the routed pairs by owner, publish the counts, wait for everybody's, store
        rows + metadata into the owners' receive arrays, signal) -> recv_ready (wait for all
        rows, build the table of return addresses) -> local fused_moe on the received rows, whose
        second GEMM stores every weighted row as bf16 straight into the source rank's `back`
        array and whose last CTA signals completion -> wait_combine (wait for all returns,
        ordered k-sum).
    fused=False: the same step from single-purpose kernels (plan, publish, barrier, dispatch,
        barrier, local operator, return, barrier, combine), thirteen launches.

    fp8_wire (fused step with an fp8 quant mode; default on): the token rows are quantised once on
        the sending rank (the operator's own quantisation, as a call of its own) and cross NVLink as
        e4m3 rows + scales, half the bytes of bf16; the owner hands them to the operator as
        pre-quantised activations.  Bit-identical to sending bf16 rows; one more launch.

    dedup (fused step; default on from four experts per token): one row per (token, owner rank)
        instead of per (token, expert).  The owner receives the token's K-wide id / weight / return
        lists (-1 where the expert lives elsewhere) and its operator runs with K experts per row.
        Bit-identical to one row per pair.

    Arithmetic in both: each (token, k) partial row crosses NVLink as bf16 and the k-sum is f32 with
    one more rounding -- the operator's partial_dtype = bf16 contract.
    Every wait is a bounded spin; a rank that never arrives shows up in `status` instead of
    hanging the GPU.
    """

    def __init__(self, num_experts: int, world: int, rank: int, traits, w1_local, w2_local,
                 w1_scale=None, w2_scale=None, *, tokens_per_rank: int, topk: int, hidden: int, group=None,
                 fused: bool = True, fp8_wire: Optional[bool] = None, dedup: Optional[bool] = None):
        import copy
        import ctypes
        import os
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        import torch.distributed._symmetric_memory as symm
        from . import api
        if num_experts % world:
            raise ValueError("experts must divide evenly over ranks")
        self.api = api
        self.fused = bool(fused) and world <= 16
        self.traits = copy.copy(traits)
        if self.fused:
            self.traits.partial_dtype = "bf16"
        is_fp8 = self.traits.quant != "none"
        self.fp8_wire = self.fused and is_fp8 and hidden % 16 == 0 and (fp8_wire is None or bool(fp8_wire))
        self.dedup = self.fused and (topk >= 4 if dedup is None else bool(dedup))
        self.E, self.world, self.rank = num_experts, world, rank
        self.e_local = num_experts // world
        self.T, self.K, self.H = tokens_per_rank, topk, hidden
        dev = w1_local.device
        R = tokens_per_rank * topk
        # rows this rank can receive: every routed pair of every rank, or every token once
        recv_cap = tokens_per_rank * world if self.dedup else R * world
        kw = topk if self.dedup else 1          # width of the per-row id / weight / return lists

        def al(n):
            return (n + 255) // 256 * 256
        lay = api.EpLayout()
        off = 0
        row_bytes = hidden if self.fp8_wire else hidden * 2
        scale_bytes = api.quant_scale_row_bytes(self.traits.quant, hidden) if self.fp8_wire else 0
        self.row_bytes, self.scale_row_bytes = row_bytes, scale_bytes
        for name, nbytes in (("flags", world * 4), ("flags_dispatch", world * 4), ("flags_return", world * 4),
                             ("matrix", world * world * 4),
                             ("rows", recv_cap * row_bytes), ("row_scales", recv_cap * scale_bytes),
                             ("ids", recv_cap * kw * 4), ("weights", recv_cap * kw * 4),
                             ("src", recv_cap * max(2, kw) * 4), ("src_rank", recv_cap * 4),
                             ("back", R * hidden * 2)):
            setattr(lay, name, off)
            off = al(off + nbytes)
        lay.recv_cap, lay.send_cap = recv_cap, R
        self.lay = lay
        group = group or dist.group.WORLD
        self.buf = symm.empty(off, dtype=torch.uint8, device=dev)
        self.buf.zero_()
        torch.cuda.synchronize()
        self.hdl = symm.rendezvous(self.buf, group)
        self.peer_base = torch.tensor(list(self.hdl.buffer_ptrs), dtype=torch.int64, device=dev)
        dist.barrier(group=group)

        def view(name, n, dt):
            o = getattr(lay, name)
            return self.buf[o:o + n * torch.empty((), dtype=dt).element_size()].view(dt)
        if self.fp8_wire:
            self.rows = view("rows", recv_cap * hidden, torch.uint8).view(recv_cap, hidden)
            self.row_scales = view("row_scales", recv_cap * scale_bytes, torch.uint8).view(recv_cap, scale_bytes)
            self.xq = torch.empty(tokens_per_rank, hidden, dtype=torch.uint8, device=dev)
            self.xq_scale = torch.empty(tokens_per_rank, scale_bytes, dtype=torch.uint8, device=dev)
        else:
            self.rows = view("rows", recv_cap * hidden, torch.bfloat16).view(recv_cap, hidden)
            self.row_scales = None
        self.ids = view("ids", recv_cap * kw, torch.int32).view(recv_cap, kw)
        self.wts = view("weights", recv_cap * kw, torch.float32).view(recv_cap, kw)
        self.back = view("back", R * hidden, torch.bfloat16).view(R, hidden)
        self.order = torch.empty(R, dtype=torch.int32, device=dev)
        self.inv = torch.empty(R, dtype=torch.int32, device=dev)
        self.cum = torch.zeros(world + 1, dtype=torch.int32, device=dev)
        self.scratch = torch.empty(R, dtype=torch.int32, device=dev)
        self.n_recv = torch.zeros(1, dtype=torch.int32, device=dev)
        self.status = torch.zeros(1, dtype=torch.int32, device=dev)
        self.out_rows = torch.empty(recv_cap, hidden, dtype=torch.bfloat16, device=dev)
        self.args = api.FusedMoeArgs(a=self.rows, g=w1_local, d=w2_local, topk_ids=self.ids,
                                     topk_weight=self.wts, o=self.out_rows, g_scale=w1_scale,
                                     d_scale=w2_scale, num_tokens_dev=self.n_recv,
                                     expected_tokens=tokens_per_rank if self.dedup else R,
                                     a_scale=self.row_scales)
        self.epoch_dev = torch.zeros(1, dtype=torch.int32, device=dev)
        if self.fused:
            # fused step: the epoch starts at 1 and is advanced on the device by wait_combine
            self.epoch_dev.fill_(1)
            self.send_scratch = torch.zeros(int(api.lib().fmoe_ep_send_scratch_words(tokens_per_rank, topk, world)),
                                            dtype=torch.int32, device=dev)
            self.row_ptrs = torch.zeros(recv_cap * kw, dtype=torch.int64, device=dev)
            self.args.partial_row_ptrs = self.row_ptrs
            self.args.done_flag_addrs = (self.peer_base + (lay.flags_return + 4 * rank)).contiguous()
            self.args.done_flag_value = self.epoch_dev
            self.args.done_counter = torch.zeros(1, dtype=torch.int32, device=dev)
        self.args.workspace = torch.empty(api.fused_moe_workspace_size(self.traits, self.args), dtype=torch.uint8,
                                          device=dev)
        self.barrier_timeout_ms = 0          # 0 = the library default (about four seconds)
        self.trace = None                    # set to [] to collect (phase, cuda event) marks
        self._ctypes = ctypes
        ops = api.launches_per_run(self.traits, self.args)
        self.launches_per_step = (3 + ops + (1 if self.fp8_wire else 0)) if self.fused else (8 + ops)
        torch.cuda.synchronize()
        dist.barrier(group=group)

    def _barrier(self, stream):
        # the epoch is a device-side counter, so the launch arguments never change
        self.api._check(self.api.lib().fmoe_ep_barrier(self.peer_base.data_ptr(), self._ctypes.byref(self.lay),
                                                       self.rank, self.world, 0, self.epoch_dev.data_ptr(),
                                                       self.status.data_ptr(), self.barrier_timeout_ms, stream))

    def _forward_fused(self, x, topk_ids, topk_weight, out):
        api, lib, by = self.api, self.api.lib(), self._ctypes.byref
        T, K, H, G = self.T, self.K, self.H, self.world
        st = api._stream_ptr(None)
        pb = self.peer_base.data_ptr()
        if out is None:
            out = torch.empty(T, H, dtype=torch.bfloat16, device=x.device)
        self._mark("start")
        if self.fp8_wire or self.dedup:
            if self.fp8_wire:
                api.quantise_rows(x, self.traits.quant, self.xq, self.xq_scale)
                rows, scales = self.xq.data_ptr(), self.xq_scale.data_ptr()
            else:
                rows, scales = x.data_ptr(), None
            send = lib.fmoe_ep_send_rows_dedup if self.dedup else lib.fmoe_ep_send_rows
            api._check(send(rows, self.row_bytes, scales, self.scale_row_bytes, topk_ids.data_ptr(),
                            topk_weight.data_ptr(), T, K, self.e_local, pb, by(self.lay), self.rank, G,
                            self.send_scratch.data_ptr(), self.epoch_dev.data_ptr(), self.n_recv.data_ptr(),
                            self.status.data_ptr(), self.barrier_timeout_ms, st))
        else:
            api._check(lib.fmoe_ep_send(x.data_ptr(), topk_ids.data_ptr(), topk_weight.data_ptr(), T, K, H,
                                        self.e_local, pb, by(self.lay), self.rank, G, self.send_scratch.data_ptr(),
                                        self.epoch_dev.data_ptr(), self.n_recv.data_ptr(), self.status.data_ptr(),
                                        self.barrier_timeout_ms, st))
        self._mark("send")
        if self.dedup:
            api._check(lib.fmoe_ep_recv_ready_dedup(H, K, self.n_recv.data_ptr(), pb, by(self.lay), self.rank, G,
                                                    self.epoch_dev.data_ptr(), self.row_ptrs.data_ptr(),
                                                    self.send_scratch.data_ptr(), self.status.data_ptr(),
                                                    self.barrier_timeout_ms, st))
        else:
            api._check(lib.fmoe_ep_recv_ready(H, self.n_recv.data_ptr(), pb, by(self.lay), self.rank, G,
                                              self.epoch_dev.data_ptr(), self.row_ptrs.data_ptr(),
                                              self.send_scratch.data_ptr(), self.status.data_ptr(),
                                              self.barrier_timeout_ms, st))
        self._mark("recv_ready")
        api.fused_moe(self.traits, self.args)
        self._mark("local_moe")
        api._check(lib.fmoe_ep_wait_combine(topk_ids.data_ptr(), T, K, H, self.E, pb, by(self.lay), self.rank, G,
                                            self.epoch_dev.data_ptr(), self.send_scratch.data_ptr(), out.data_ptr(),
                                            self.status.data_ptr(), self.barrier_timeout_ms, st))
        self._mark("wait_combine")
        return out

    def forward(self, x: torch.Tensor, topk_ids: torch.Tensor, topk_weight: torch.Tensor,
                out: Optional[torch.Tensor] = None) -> torch.Tensor:
        api, lib, by = self.api, self.api.lib(), self._ctypes.byref
        T, K, H, G = self.T, self.K, self.H, self.world
        assert x.shape == (T, H) and topk_ids.shape == (T, K)
        if self.fused:
            return self._forward_fused(x, topk_ids, topk_weight, out)
        st = api._stream_ptr(None)
        pb = self.peer_base.data_ptr()
        self._mark("start")
        api._check(lib.fmoe_ep_plan(topk_ids.data_ptr(), T, K, self.e_local, G, self.order.data_ptr(),
                                    self.inv.data_ptr(), self.cum.data_ptr(), self.scratch.data_ptr(), st))
        api._check(lib.fmoe_ep_publish(self.cum.data_ptr(), pb, by(self.lay), self.rank, G, st))
        self._mark("plan")
        self._barrier(st)
        self._mark("barrier1")
        api._check(lib.fmoe_ep_dispatch(x.data_ptr(), topk_ids.data_ptr(), topk_weight.data_ptr(), T, K, H,
                                        self.e_local, self.order.data_ptr(), self.cum.data_ptr(), pb,
                                        by(self.lay), self.rank, G, self.n_recv.data_ptr(), st))
        self._mark("dispatch")
        self._barrier(st)
        self._mark("barrier2")
        api.fused_moe(self.traits, self.args)
        self._mark("local_moe")
        api._check(lib.fmoe_ep_return(self.out_rows.data_ptr(), H, self.n_recv.data_ptr(), pb, by(self.lay),
                                      self.rank, G, st))
        self._mark("return")
        self._barrier(st)
        self._mark("barrier3")
        res = api.combine_rows(self.back, self.inv, T, K, out=out)
        self._mark("combine")
        return res

    def _mark(self, name):
        if self.trace is not None:
            ev = torch.cuda.Event(enable_timing=True)
            ev.record()
            self.trace.append((name, ev))

    def check_status(self) -> int:
        torch.cuda.synchronize()
        return int(self.status.item()) | self.api.check_status(self.args.workspace)
