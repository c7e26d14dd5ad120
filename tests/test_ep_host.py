"""Host-side logic of the expert-parallel wrapper on CPU ranks (gloo, world size 2 and 4):
destination planning, count exchange, all-to-all dispatch / return and the ordered
combine.  The two CUDA kernels and the local operator are replaced by CPU stand-ins (the
oracle plays the local operator), so no GPU is needed."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import oracle as O
from therock_b200 import ep


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _cpu_gather(src, row_ids):
    return src[row_ids.long()].contiguous()


def _cpu_combine(rows, index, T, K):
    H = rows.shape[1]
    acc = torch.zeros(T, H, dtype=torch.float32)
    idx = index.view(T, K).long()
    for k in range(K):
        m = idx[:, k] >= 0
        acc[m] += rows[idx[m, k]].float()
    return acc.to(torch.bfloat16)


def _bits(t):
    return t.view(torch.int16).numpy().view(np.uint16)


def _worker(rank, world, port, T, H, I, E, K, quant, drop, ret, dedup=False):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        d = O.make_inputs(T, H, I, E, K, quant, "softmax", seed=3)
        if drop:
            d["topk_ids"][::5, 0] = -1
        e_local = E // world
        lo = rank * e_local
        w1 = d["w1"][lo:lo + e_local]
        w2 = d["w2"][lo:lo + e_local]
        s1 = None if quant == 0 else d["w1_scale"][lo:lo + e_local]
        s2 = None if quant == 0 else d["w2_scale"][lo:lo + e_local]

        def local_moe(x_rows, ids_local, w_local):
            out = O.fused_moe(_bits(x_rows), w1, w2, ids_local.numpy(), w_local.numpy(), quant, s1, s2, n_threads=2)
            return torch.from_numpy(out.view(np.int16)).view(torch.bfloat16)

        t_local = T // world
        sl = slice(rank * t_local, (rank + 1) * t_local)
        x = torch.from_numpy(d["x"][sl].view(np.int16)).view(torch.bfloat16)
        ids = torch.from_numpy(d["topk_ids"][sl].copy())
        wts = torch.from_numpy(d["topk_w"][sl].copy())
        moe = ep.ExpertParallelMoE(E, world, rank, local_moe, gather=_cpu_gather, combine=_cpu_combine,
                                   dedup=dedup)
        out = moe.forward(x, ids, wts)
        # partial rows travel as bf16 before the k-sum: the oracle's bf16-partial mode is the
        # reference (de-duplicated dispatch sums a rank's experts in f32 first: looser bound there)
        ref = O.fused_moe(d["x"], d["w1"], d["w2"], d["topk_ids"], d["topk_w"], quant, d["w1_scale"], d["w2_scale"],
                          sel=np.arange(sl.start, sl.stop, dtype=np.int32), partial_bf16=not dedup)
        g, r = O.bf16_to_f32(_bits(out)), O.bf16_to_f32(ref)
        bound = 5e-3 if dedup else (2e-3 if quant == 0 else 4e-2)
        ok = np.allclose(g, r, rtol=1e-2, atol=1e-2) and np.linalg.norm(g - r) <= bound * np.linalg.norm(r)
        ret[rank] = bool(ok)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,quant,drop", [(2, 0, False), (2, 1, True), (4, 0, True)])
def test_expert_parallel_matches_single_rank_oracle(world, quant, drop):
    ctx = mp.get_context("spawn")
    ret = ctx.Manager().dict()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, 64, 256, 128, 8, 2, quant, drop, ret))
             for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(180)
        assert p.exitcode == 0
    assert all(ret.get(r) for r in range(world)), dict(ret)


@pytest.mark.parametrize("world,quant,K", [(2, 0, 4), (4, 1, 3)])
def test_deduplicated_dispatch_matches_single_rank_oracle(world, quant, K):
    ctx = mp.get_context("spawn")
    ret = ctx.Manager().dict()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, 64, 256, 128, 8, K, quant, True, ret, True))
             for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(180)
        assert p.exitcode == 0
    assert all(ret.get(r) for r in range(world)), dict(ret)


def test_dedup_plan_sends_one_row_per_token_and_rank():
    ids = torch.tensor([[0, 1, 5], [4, 6, 7], [2, 9, -1], [3, 4, 0]], dtype=torch.int32)   # 8 experts, 2 ranks
    w = torch.arange(12, dtype=torch.float32).reshape(4, 3) + 1
    # world = 2 without a process group: only the local arithmetic (the count exchange needs ranks)
    T, K, world, epr = 4, 3, 2, 4
    dest = torch.where((ids >= 0) & (ids < 8), ids.long() // epr, torch.full_like(ids.long(), world))
    hit = torch.zeros(T, world + 1, dtype=torch.bool).scatter_(1, dest, True)[:, :world]
    assert hit.tolist() == [[True, True], [False, True], [True, False], [True, True]]
    assert int(hit.sum()) == 6 < int(((ids >= 0) & (ids < 8)).sum())       # 6 rows instead of 10 pairs
    single = ep.plan_dispatch_dedup(ids, w, experts_per_rank=8, world=1)
    assert single.n_send == 4 and single.send_counts == [4] and single.index.tolist() == [0, 1, 2, 3]
    assert single.ids.tolist() == [[0, 1, 5], [4, 6, 7], [2, -1, -1], [3, 4, 0]]
    assert single.weights[2].tolist() == [7.0, 0.0, 0.0]


def test_plan_dispatch_single_rank_is_stable_grouping():
    ids = torch.tensor([[3, 0], [1, 2], [0, 3], [2, -1]], dtype=torch.int32)
    plan = ep.plan_dispatch(ids, experts_per_rank=4, world=1)
    assert plan.n_send == 7 and plan.send_counts == [7] and plan.recv_counts == [7]
    assert plan.order.tolist() == [0, 1, 2, 3, 4, 5, 6]
    assert plan.inv_index.tolist() == [0, 1, 2, 3, 4, 5, 6, -1]


def test_plan_dispatch_groups_by_destination():
    ids = torch.tensor([[3, 0], [1, 2], [0, 3], [2, 9]], dtype=torch.int32)
    # world=2 without a process group: exercise only the local arithmetic
    flat = ids.reshape(-1).long()
    dest = torch.where((flat >= 0) & (flat < 4), flat // 2, torch.full_like(flat, 2))
    order = torch.argsort(dest, stable=True)[:7]
    assert order.tolist() == [1, 2, 4, 0, 3, 5, 6]     # rank 0 pairs first, original order kept


def _timeout_worker(rank, world, port, ret):
    """Rank 0 runs a step with a 2 s limit; rank 1 joins the group but never enters the step
    (a rank that stalls between steps), then leaves."""
    import time
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        if rank == 1:
            time.sleep(8.0)
            ret[rank] = "stalled"
            return
        moe = ep.ExpertParallelMoE(4, world, rank, lambda x, i, w: x, gather=_cpu_gather, combine=_cpu_combine,
                                   timeout_s=2.0)
        x = torch.zeros(8, 64, dtype=torch.bfloat16)
        ids = torch.zeros(8, 2, dtype=torch.int32)
        wts = torch.ones(8, 2)
        t0 = time.time()
        try:
            moe.forward(x, ids, wts)
            ret[rank] = "no error"
        except ep.ExpertParallelTimeout as exc:
            ret[rank] = f"timeout after {time.time() - t0:.1f}s: {str(exc)[:60]}"
    finally:
        try:
            dist.destroy_process_group()
        except Exception:
            pass


def test_missing_rank_raises_a_timeout_instead_of_blocking():
    """Failure detection of the collective transport, injected on the host: one rank never
    enters the step; the other must get ExpertParallelTimeout within its own short limit."""
    ctx = mp.get_context("spawn")
    ret = ctx.Manager().dict()
    port = _free_port()
    procs = [ctx.Process(target=_timeout_worker, args=(r, 2, port, ret)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(60)
    assert str(ret.get(0, "")).startswith("timeout after"), dict(ret)
    assert float(str(ret[0]).split()[2].rstrip("s:")) < 7.0
