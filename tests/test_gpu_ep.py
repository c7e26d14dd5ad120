"""Expert-parallel wrapper on real GPUs: the CUDA pack / combine kernels and the local
operator, on one GPU (world size 1) and, where the box has them, on two GPUs over NCCL."""
import os
import socket

import numpy as np
import pytest
import torch

from oracle import oracle as O
from tests.util import QUANT_NAME, bf16_dev, out_bits, to_dev, traits_for

pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _close(got_bits, ref_bits, quant):
    """The operator's own tolerances.  The expert-parallel paths return each (token, k) partial
    row as bf16, so their reference is the oracle's bf16-partial mode (partial_bf16=True)."""
    g, r = O.bf16_to_f32(got_bits), O.bf16_to_f32(ref_bits)
    return (np.allclose(g, r, rtol=1e-2, atol=1e-2) or quant != 0) and \
        np.linalg.norm(g - r) <= (2e-3 if quant == 0 else 4e-2) * np.linalg.norm(r)


def _rank_forward(d, rank, world, device, dedup=False):
    from therock_b200 import ep
    quant = d["quant"]
    E = d["w1"].shape[0]
    e_local = E // world
    lo = rank * e_local
    if quant == 0:
        w1, w2 = bf16_dev(d["w1"][lo:lo + e_local], device), bf16_dev(d["w2"][lo:lo + e_local], device)
        s1 = s2 = None
    else:
        w1, w2 = to_dev(d["w1"][lo:lo + e_local], device=device), to_dev(d["w2"][lo:lo + e_local], device=device)
        s1 = to_dev(d["w1_scale"][lo:lo + e_local], device=device)
        s2 = to_dev(d["w2_scale"][lo:lo + e_local], device=device)
    T = d["x"].shape[0]
    t_local = T // world
    sl = slice(rank * t_local, (rank + 1) * t_local)
    local = ep.make_local_moe(traits_for(quant), w1, w2, s1, s2)
    moe = ep.ExpertParallelMoE(E, world, rank, local, dedup=dedup)
    out = moe.forward(bf16_dev(d["x"][sl], device), to_dev(d["topk_ids"][sl], device=device),
                      to_dev(d["topk_w"][sl], device=device))
    torch.cuda.synchronize()
    return out_bits(out), sl


@pytest.mark.parametrize("quant", [0, 1])
def test_single_rank_expert_parallel_path(quant):
    d = O.make_inputs(200, 512, 256, 8, 2, quant, "softmax", seed=21)
    d["topk_ids"][::9, 1] = -1
    got, _ = _rank_forward(d, 0, 1, "cuda:0")
    ref = O.fused_moe(d["x"], d["w1"], d["w2"], d["topk_ids"], d["topk_w"], quant, d["w1_scale"], d["w2_scale"],
                      partial_bf16=True)
    assert _close(got, ref, quant)


@pytest.mark.parametrize("quant", [0, 1])
def test_single_rank_deduplicated_dispatch(quant):
    # one row per token with its K-wide id list (invalid ids stay -1): the CUDA gather,
    # operator and combine kernels behind the de-duplicated plan
    d = O.make_inputs(200, 512, 256, 8, 3, quant, "softmax", seed=22)
    d["topk_ids"][::7, 2] = -1
    got, _ = _rank_forward(d, 0, 1, "cuda:0", dedup=True)
    # one rank owns every expert: the token's K terms are summed in f32 inside the operator
    ref = O.fused_moe(d["x"], d["w1"], d["w2"], d["topk_ids"], d["topk_w"], quant, d["w1_scale"], d["w2_scale"])
    assert _close(got, ref, quant)


def _peer_worker(rank, world, port, quant, ret, fused=True):
    import torch.distributed as dist
    from therock_b200 import ep
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0",
                      TORCH_SYMM_MEM_DISABLE_MULTICAST="1")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        T, H, I, E, K = 256, 512, 256, 8, 2
        d = O.make_inputs(T, H, I, E, K, quant, "softmax", seed=23)
        d["topk_ids"][::13, 0] = -1
        e_local = E // world
        lo = rank * e_local
        if quant == 0:
            w1, w2, s1, s2 = bf16_dev(d["w1"][lo:lo + e_local], dev), bf16_dev(d["w2"][lo:lo + e_local], dev), None, None
        else:
            w1, w2 = to_dev(d["w1"][lo:lo + e_local], device=dev), to_dev(d["w2"][lo:lo + e_local], device=dev)
            s1, s2 = to_dev(d["w1_scale"][lo:lo + e_local], device=dev), to_dev(d["w2_scale"][lo:lo + e_local], device=dev)
        t_local = T // world
        sl = slice(rank * t_local, (rank + 1) * t_local)
        moe = ep.PeerExpertParallelMoE(E, world, rank, traits_for(quant), w1, w2, s1, s2,
                                       tokens_per_rank=t_local, topk=K, hidden=H, fused=fused)
        x, ids, w = bf16_dev(d["x"][sl], dev), to_dev(d["topk_ids"][sl], device=dev), to_dev(d["topk_w"][sl], device=dev)
        ref = O.fused_moe(d["x"], d["w1"], d["w2"], d["topk_ids"], d["topk_w"], quant, d["w1_scale"], d["w2_scale"],
                          sel=np.arange(sl.start, sl.stop, dtype=np.int32), partial_bf16=True)
        ok = True
        for _ in range(3):      # repeated steps reuse the same peer buffers
            out = moe.forward(x, ids, w)
            ok = ok and moe.check_status() == 0 and bool(_close(out_bits(out), ref, quant))
        ret[rank] = ok
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("fused", [True, False])
@pytest.mark.parametrize("quant", [0, 1, 3])
def test_peer_memory_step_with_a_single_rank(quant, fused):
    """World size 1: the whole peer-memory step (fused: send, recv_ready, the operator storing
    its partial rows through the return-address table and signalling, wait_combine) on one GPU,
    where every flag this rank waits for is its own."""
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    ret = ctx.Manager().dict()
    p = ctx.Process(target=_peer_worker, args=(0, 1, _free_port(), quant, ret, fused))
    p.start()
    p.join(300)
    assert p.exitcode == 0
    assert ret.get(0), dict(ret)


@pytest.mark.parametrize("fused", [True, False])
@pytest.mark.parametrize("quant", [0, 1])
def test_two_gpu_peer_memory_expert_parallel(quant, fused):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    ret = ctx.Manager().dict()
    port = _free_port()
    procs = [ctx.Process(target=_peer_worker, args=(r, 2, port, quant, ret, fused)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(300)
        assert p.exitcode == 0
    assert all(ret.get(r) for r in range(2)), dict(ret)


def _worker(rank, world, port, quant, ret, dedup=False):
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        # de-duplicated: K = 5 exceeds the 4 experts a rank owns, so the local operator sees
        # K-wide id lists with more columns than it has experts
        d = O.make_inputs(256, 512, 256, 8, 5 if dedup else 2, quant, "softmax", seed=22)
        got, sl = _rank_forward(d, rank, world, f"cuda:{rank}", dedup=dedup)
        ref = O.fused_moe(d["x"], d["w1"], d["w2"], d["topk_ids"], d["topk_w"], quant, d["w1_scale"], d["w2_scale"],
                          sel=np.arange(sl.start, sl.stop, dtype=np.int32), partial_bf16=not dedup)
        ret[rank] = bool(_close(got, ref, quant)) if not dedup else bool(
            np.linalg.norm(O.bf16_to_f32(got) - O.bf16_to_f32(ref)) <= 4e-2 * np.linalg.norm(O.bf16_to_f32(ref)))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("quant,dedup", [(0, False), (1, False), (1, True)])
def test_two_gpu_expert_parallel(quant, dedup):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    ret = ctx.Manager().dict()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, quant, ret, dedup)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(300)
        assert p.exitcode == 0
    assert all(ret.get(r) for r in range(2)), dict(ret)


def test_barrier_wait_is_bounded_when_a_rank_never_arrives():
    """Failure detection without a fault: a two-rank barrier in which the second rank never
    writes its flag.  Both "ranks" are buffers on this one GPU; the kernel must give up after
    the timeout, report the missing rank in the status word and leave the context usable."""
    import ctypes
    from therock_b200 import api
    dev = "cuda:0"
    lay = api.EpLayout()
    lay.flags, lay.matrix = 0, 256
    mine = torch.zeros(1024, dtype=torch.uint8, device=dev)
    theirs = torch.zeros(1024, dtype=torch.uint8, device=dev)
    peer_base = torch.tensor([mine.data_ptr(), theirs.data_ptr()], dtype=torch.int64, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    st = torch.cuda.current_stream().cuda_stream
    rc = api.lib().fmoe_ep_barrier(peer_base.data_ptr(), ctypes.byref(lay), 0, 2, 1, None, status.data_ptr(), 50, st)
    assert rc == 0
    torch.cuda.synchronize()
    assert int(status.item()) == (0x300 | 1)                       # rank 1 was never seen
    assert int(theirs[:8].view(torch.int32)[0].item()) == 1        # our own arrival was published
    # the context is still healthy and a satisfied barrier passes
    status.zero_()
    mine[:8].view(torch.int32)[1] = 2                               # pretend rank 1 arrived at epoch 2
    rc = api.lib().fmoe_ep_barrier(peer_base.data_ptr(), ctypes.byref(lay), 0, 2, 2, None, status.data_ptr(), 50, st)
    torch.cuda.synchronize()
    assert rc == 0 and int(status.item()) == 0
    # device-side epoch counter: the kernel advances it itself (1 -> 2 -> 3)
    counter = torch.tensor([2], dtype=torch.int32, device=dev)
    mine[:8].view(torch.int32)[1] = 3
    rc = api.lib().fmoe_ep_barrier(peer_base.data_ptr(), ctypes.byref(lay), 0, 2, 0, counter.data_ptr(),
                                   status.data_ptr(), 50, st)
    torch.cuda.synchronize()
    assert rc == 0 and int(status.item()) == 0 and int(counter.item()) == 3
    assert int(theirs[:8].view(torch.int32)[0].item()) == 3


def _fake_two_rank_layout(dev, T, K, H, kw=1):
    """Two full peer buffers on one GPU: rank 0 is driven by the test, rank 1 never acts.
    kw: width of the per-row id / weight / return lists (K in the de-duplicated step)."""
    from therock_b200 import api
    lay = api.EpLayout()
    R, world = T * K, 2
    recv_cap, off = R * world, 0
    for name, nbytes in (("flags", 8), ("flags_dispatch", 8), ("flags_return", 8), ("matrix", 16),
                         ("rows", recv_cap * H * 2), ("row_scales", 256), ("ids", recv_cap * kw * 4),
                         ("weights", recv_cap * kw * 4), ("src", recv_cap * max(2, kw) * 4),
                         ("src_rank", recv_cap * 4), ("back", R * H * 2)):
        setattr(lay, name, off)
        off = (off + nbytes + 255) // 256 * 256
    lay.recv_cap, lay.send_cap = recv_cap, R
    mine = torch.zeros(off, dtype=torch.uint8, device=dev)
    theirs = torch.zeros(off, dtype=torch.uint8, device=dev)
    peer_base = torch.tensor([mine.data_ptr(), theirs.data_ptr()], dtype=torch.int64, device=dev)
    return lay, mine, theirs, peer_base


@pytest.mark.parametrize("dedup", [False, True])
def test_fused_step_waits_are_bounded_when_a_rank_never_arrives(dedup):
    """Failure detection for the fused kernels without a fault: rank 1 of a two-rank step never
    writes any flag.  Each of the three kernels (both forms of the send and of recv_ready) must
    give up after its 50 ms limit, report rank 1 in the status word and return, leaving the
    context usable."""
    import ctypes
    from therock_b200 import api
    dev = "cuda:0"
    T, K, H, e_local = 64, 2, 256, 4
    lay, mine, theirs, peer_base = _fake_two_rank_layout(dev, T, K, H, kw=K if dedup else 1)
    lib, by = api.lib(), ctypes.byref
    st = torch.cuda.current_stream().cuda_stream
    d = O.make_inputs(T, H, 128, 2 * e_local, K, 0, "softmax", seed=41)
    x, ids, w = bf16_dev(d["x"], dev), to_dev(d["topk_ids"], device=dev), to_dev(d["topk_w"], device=dev)
    epoch = torch.ones(1, dtype=torch.int32, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    n_recv = torch.zeros(1, dtype=torch.int32, device=dev)
    scratch = torch.zeros(int(lib.fmoe_ep_send_scratch_words(T, K, 2)), dtype=torch.int32, device=dev)
    if dedup:
        rc = lib.fmoe_ep_send_rows_dedup(x.data_ptr(), 2 * H, None, 0, ids.data_ptr(), w.data_ptr(), T, K, e_local,
                                         peer_base.data_ptr(), by(lay), 0, 2, scratch.data_ptr(), epoch.data_ptr(),
                                         n_recv.data_ptr(), status.data_ptr(), 50, st)
    else:
        rc = lib.fmoe_ep_send(x.data_ptr(), ids.data_ptr(), w.data_ptr(), T, K, H, e_local, peer_base.data_ptr(),
                              by(lay), 0, 2, scratch.data_ptr(), epoch.data_ptr(), n_recv.data_ptr(),
                              status.data_ptr(), 50, st)
    assert rc == 0
    torch.cuda.synchronize()
    assert int(status.item()) == (0x300 | 1)
    # our own counts and the completion flag were still published to the silent rank
    assert int(theirs[lay.flags:lay.flags + 4].view(torch.int32).item()) == 1
    assert int(theirs[lay.flags_dispatch:lay.flags_dispatch + 4].view(torch.int32).item()) == 1
    assert int(scratch[:2].abs().sum().item()) == 0                  # the kernel's own counters are back at zero
    status.zero_()
    row_ptrs = torch.zeros(int(lay.recv_cap) * K, dtype=torch.int64, device=dev)
    if dedup:
        rc = lib.fmoe_ep_recv_ready_dedup(H, K, n_recv.data_ptr(), peer_base.data_ptr(), by(lay), 0, 2,
                                          epoch.data_ptr(), row_ptrs.data_ptr(), scratch.data_ptr(),
                                          status.data_ptr(), 50, st)
    else:
        rc = lib.fmoe_ep_recv_ready(H, n_recv.data_ptr(), peer_base.data_ptr(), by(lay), 0, 2, epoch.data_ptr(),
                                    row_ptrs.data_ptr(), scratch.data_ptr(), status.data_ptr(), 50, st)
    torch.cuda.synchronize()
    assert rc == 0 and int(status.item()) == (0x300 | 1)
    status.zero_()
    out = torch.empty(T, H, dtype=torch.bfloat16, device=dev)
    # this rank's own operator would have signalled its returns; rank 1 never does
    mine[lay.flags_return:lay.flags_return + 4].view(torch.int32)[0] = 1
    rc = lib.fmoe_ep_wait_combine(ids.data_ptr(), T, K, H, 2 * e_local, peer_base.data_ptr(), by(lay), 0, 2,
                                  epoch.data_ptr(), scratch.data_ptr(), out.data_ptr(), status.data_ptr(), 50, st)
    torch.cuda.synchronize()
    assert rc == 0 and int(status.item()) == (0x300 | 1)
    assert int(epoch.item()) == 2 and int(scratch[5].item()) == 0    # the step was closed all the same
    # the context is healthy: a plain operator call still works
    from tests.util import run_gpu
    run_gpu(d)


def _stress_worker(rank, world, port, quant, steps, ret, dedup=None, K=2):
    """Many steps with fresh routing and activations every step, the fused step and the
    single-purpose kernels side by side: both return bf16 partial rows and add them in k order,
    so their outputs must agree bit for bit; a race between steps (a flag, a count or a row
    arriving in the wrong epoch) would show up as a difference."""
    import torch.distributed as dist
    from therock_b200 import ep
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0",
                      TORCH_SYMM_MEM_DISABLE_MULTICAST="1")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        T, H, I, E = 192 * world, 512, 256, 8
        d = O.make_inputs(T, H, I, E, K, quant, "softmax", seed=29)
        e_local, t_local = E // world, T // world
        lo = rank * e_local
        if quant == 0:
            w1, w2, s1, s2 = bf16_dev(d["w1"][lo:lo + e_local], dev), bf16_dev(d["w2"][lo:lo + e_local], dev), None, None
        else:
            w1, w2 = to_dev(d["w1"][lo:lo + e_local], device=dev), to_dev(d["w2"][lo:lo + e_local], device=dev)
            s1, s2 = to_dev(d["w1_scale"][lo:lo + e_local], device=dev), to_dev(d["w2_scale"][lo:lo + e_local], device=dev)
        mk = lambda fused: ep.PeerExpertParallelMoE(E, world, rank, traits_for(quant), w1, w2, s1, s2,
                                                    tokens_per_rank=t_local, topk=K, hidden=H, fused=fused,
                                                    dedup=dedup)
        fused, plain = mk(True), mk(False)
        g = torch.Generator(device=dev)
        g.manual_seed(1000 + rank)
        bad = 0
        for step in range(steps):
            x = torch.randn(t_local, H, generator=g, device=dev).to(torch.bfloat16)
            logits = torch.randn(t_local, E, generator=g, device=dev)
            if step % 5 == 4:
                logits[:, : E // 2] += 4.0          # skewed routing: one half of the ranks gets almost everything
            w, ids = torch.topk(torch.softmax(logits, -1), K, dim=-1)
            ids = ids.to(torch.int32).contiguous()
            if step % 7 == 3:
                ids[::11, 0] = -1                   # dropped pairs
            w = (w / w.sum(-1, keepdim=True)).float().contiguous()
            a = fused.forward(x, ids, w).clone()
            b = plain.forward(x, ids, w).clone()
            bad += int((a.view(torch.int16) != b.view(torch.int16)).sum().item())
        ok = bad == 0 and fused.check_status() == 0 and plain.check_status() == 0
        ret[rank] = bool(ok) if ok else f"{bad} differing elements, status {fused.check_status()} / {plain.check_status()}"
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("quant,dedup,K", [(0, False, 2), (1, False, 2), (3, False, 2), (0, True, 2), (3, True, 2),
                                           (1, True, 5)])
def test_fused_and_single_purpose_steps_agree_bit_for_bit_over_many_random_steps(quant, dedup, K):
    """With an fp8 quant mode the fused step also sends e4m3 rows + scales where the single-purpose
    kernels send bf16 rows, and with dedup one row per (token, owner rank) with K-wide lists
    (K = 5 of 8 experts on 2 ranks: more experts per token than a rank owns): the agreement covers
    that neither the wire format nor the de-duplication changes a bit."""
    world = 2 if torch.cuda.device_count() >= 2 else 1
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    ret = ctx.Manager().dict()
    port = _free_port()
    procs = [ctx.Process(target=_stress_worker, args=(r, world, port, quant, 40, ret, dedup, K)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(600)
        assert p.exitcode == 0
    assert all(ret.get(r) is True for r in range(world)), dict(ret)
