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
    g, r = O.bf16_to_f32(got_bits), O.bf16_to_f32(ref_bits)
    # returned partial rows are bf16: one extra rounding per term compared with fused_moe
    return (np.allclose(g, r, rtol=2e-2, atol=1e-2) or quant != 0) and \
        np.linalg.norm(g - r) <= (6e-3 if quant == 0 else 4e-2) * np.linalg.norm(r)


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
    ref = O.fused_moe(d["x"], d["w1"], d["w2"], d["topk_ids"], d["topk_w"], quant, d["w1_scale"], d["w2_scale"])
    assert _close(got, ref, quant)


@pytest.mark.parametrize("quant", [0, 1])
def test_single_rank_deduplicated_dispatch(quant):
    # one row per token with its K-wide id list (invalid ids stay -1): the CUDA gather,
    # operator and combine kernels behind the de-duplicated plan
    d = O.make_inputs(200, 512, 256, 8, 3, quant, "softmax", seed=22)
    d["topk_ids"][::7, 2] = -1
    got, _ = _rank_forward(d, 0, 1, "cuda:0", dedup=True)
    ref = O.fused_moe(d["x"], d["w1"], d["w2"], d["topk_ids"], d["topk_w"], quant, d["w1_scale"], d["w2_scale"])
    assert _close(got, ref, quant)


def _peer_worker(rank, world, port, quant, ret):
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
                                       tokens_per_rank=t_local, topk=K, hidden=H)
        x, ids, w = bf16_dev(d["x"][sl], dev), to_dev(d["topk_ids"][sl], device=dev), to_dev(d["topk_w"][sl], device=dev)
        ref = O.fused_moe(d["x"], d["w1"], d["w2"], d["topk_ids"], d["topk_w"], quant, d["w1_scale"], d["w2_scale"],
                          sel=np.arange(sl.start, sl.stop, dtype=np.int32))
        ok = True
        for _ in range(3):      # repeated steps reuse the same peer buffers
            out = moe.forward(x, ids, w)
            ok = ok and moe.check_status() == 0 and bool(_close(out_bits(out), ref, quant))
        ret[rank] = ok
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("quant", [0, 1])
def test_two_gpu_peer_memory_expert_parallel(quant):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    ret = ctx.Manager().dict()
    port = _free_port()
    procs = [ctx.Process(target=_peer_worker, args=(r, 2, port, quant, ret)) for r in range(2)]
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
        d = O.make_inputs(256, 512, 256, 8, 4 if dedup else 2, quant, "softmax", seed=22)
        got, sl = _rank_forward(d, rank, world, f"cuda:{rank}", dedup=dedup)
        ref = O.fused_moe(d["x"], d["w1"], d["w2"], d["topk_ids"], d["topk_w"], quant, d["w1_scale"], d["w2_scale"],
                          sel=np.arange(sl.start, sl.stop, dtype=np.int32))
        ret[rank] = bool(_close(got, ref, quant))
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
