"""Independent restatement of the fused-MoE contract in plain torch CPU ops.

Shares no code with oracle/: inputs come from torch's own generator, number formats from
torch's own casts (.to(torch.bfloat16), .to(torch.float8_e4m3fn)), routing from
torch.softmax / torch.sigmoid / torch.topk, the GEMMs from torch.nn.functional.linear in
float32.  Used two ways: tests/test_torch_reference.py runs it live against the C oracle, and
`python tests/golden/torch_reference.py` writes the small fixture tests/golden/torch_ref.npz that
both the oracle (CPU test) and the CUDA path (GPU test) are checked against.
"""
from __future__ import annotations

import os

import numpy as np
import torch
import torch.nn.functional as F

FP8 = torch.float8_e4m3fn
QUANT_NAMES = {0: "none", 1: "token_channel", 2: "block128", 3: "block128_ue8m0"}


def pow2_ceil(s: torch.Tensor) -> torch.Tensor:
    """Smallest power of two >= s (s > 0)."""
    m, e = torch.frexp(s)                       # s = m * 2^e, m in [0.5, 1)
    e = torch.where(m == 0.5, e - 1, e)
    return torch.ldexp(torch.ones_like(s), e)


def scales_of(amax: torch.Tensor, pow2: bool) -> torch.Tensor:
    s = amax / 448.0
    if pow2:
        s = pow2_ceil(torch.where(amax > 0, s, torch.ones_like(s)))
    return torch.where(amax > 0, s, torch.ones_like(s))


def quant_groups(a: torch.Tensor, group: int, pow2: bool = False):
    """[rows, cols] f32 -> (e4m3 values as f32 [rows, cols], scales [rows, cols/group])."""
    rows, cols = a.shape
    g = a.reshape(rows, cols // group, group)
    s = scales_of(g.abs().amax(dim=2), pow2)
    q = (g * (1.0 / s)[:, :, None]).to(FP8).to(torch.float32)
    return q.reshape(rows, cols), s


def quant_weight(wf: torch.Tensor, quant: int):
    """f32 [rows, cols] -> (stored tensor, scales or None) for one expert."""
    if quant == 0:
        return wf.to(torch.bfloat16), None
    if quant == 1:
        s = scales_of(wf.abs().amax(dim=1), False)
        return (wf * (1.0 / s)[:, None]).to(FP8), s
    rows, cols = wf.shape
    b = wf.reshape(rows // 128, 128, cols // 128, 128)
    s = scales_of(b.abs().amax(dim=(1, 3)), quant == 3)
    return (b * (1.0 / s)[:, None, :, None]).to(FP8).reshape(rows, cols), s


def route(logits: torch.Tensor, K: int, mode: str):
    p = torch.softmax(logits, dim=-1) if mode == "softmax" else torch.sigmoid(logits)
    w, ids = torch.topk(p, K, dim=-1)
    return ids.to(torch.int32), (w / w.sum(dim=-1, keepdim=True)).to(torch.float32)


def make_case(T, H, I, E, K, quant, routing, seed):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(T, H, generator=g).to(torch.bfloat16)
    logits = torch.randn(T, E, generator=g)
    ids, w = route(logits, K, routing)
    w1, w2, s1, s2 = [], [], [], []
    for _ in range(E):
        q, s = quant_weight(torch.randn(2 * I, H, generator=g) * 0.02, quant)
        w1.append(q); s1.append(s)
        q, s = quant_weight(torch.randn(H, I, generator=g) * 0.02, quant)
        w2.append(q); s2.append(s)
    return dict(x=x, ids=ids, w=w, w1=torch.stack(w1), w2=torch.stack(w2), quant=quant,
                s1=None if quant == 0 else torch.stack(s1), s2=None if quant == 0 else torch.stack(s2))


def block_linear(q, s_act, wq, s_w):
    """sum over 128-deep K blocks of (q_blk @ w_blk^T) * s_act[:, blk] * s_w[n/128, blk]."""
    out = torch.zeros(q.shape[0], wq.shape[0])
    for kb in range(q.shape[1] // 128):
        part = F.linear(q[:, kb * 128:(kb + 1) * 128], wq[:, kb * 128:(kb + 1) * 128])
        out += part * s_act[:, kb:kb + 1] * s_w[:, kb].repeat_interleave(128)[None, :]
    return out


def fused_moe(c, partial_bf16=False) -> torch.Tensor:
    """out [T, H] bf16 for a case from make_case()."""
    x, ids, w, quant = c["x"].to(torch.float32), c["ids"], c["w"], c["quant"]
    T, H = x.shape
    E, I2, _ = c["w1"].shape
    I = I2 // 2
    K = ids.shape[1]
    slots = torch.zeros(T, K, H)
    for e in range(E):
        t_idx, k_idx = torch.nonzero(ids == e, as_tuple=True)
        if t_idx.numel() == 0:
            continue
        xe = x[t_idx]
        w1, w2 = c["w1"][e].to(torch.float32), c["w2"][e].to(torch.float32)
        if quant == 0:
            gu = F.linear(xe, w1)
        elif quant == 1:
            q, s = quant_groups(xe, H)
            gu = F.linear(q, w1) * s * c["s1"][e][None, :]
        else:
            q, s = quant_groups(xe, 128, quant == 3)
            gu = block_linear(q, s, w1, c["s1"][e])
        y = (F.silu(gu[:, :I]) * gu[:, I:]).to(torch.bfloat16).to(torch.float32)
        if quant == 0:
            o = F.linear(y, w2)
        elif quant == 1:
            q, s = quant_groups(y, I)
            o = F.linear(q, w2) * s * c["s2"][e][None, :]
        else:
            q, s = quant_groups(y, 128, quant == 3)
            o = block_linear(q, s, w2, c["s2"][e])
        part = o * w[t_idx, k_idx][:, None]
        slots[t_idx, k_idx] = part.to(torch.bfloat16).to(torch.float32) if partial_bf16 else part
    acc = torch.zeros(T, H)
    for k in range(K):
        acc += slots[:, k]
    return acc.to(torch.bfloat16)


def to_numpy_case(c):
    """Bit patterns as numpy arrays (what the oracle and the C-ABI tests take)."""
    def bits16(t):
        return t.view(torch.int16).numpy().view(np.uint16).copy()

    def bits8(t):
        return t.view(torch.uint8).numpy().copy()
    q = c["quant"]
    return dict(x=bits16(c["x"]), topk_ids=c["ids"].numpy().copy(), topk_w=c["w"].numpy().copy(), quant=q,
                w1=bits16(c["w1"]) if q == 0 else bits8(c["w1"]), w2=bits16(c["w2"]) if q == 0 else bits8(c["w2"]),
                w1_scale=None if q == 0 else c["s1"].numpy().copy(), w2_scale=None if q == 0 else c["s2"].numpy().copy())


FIXTURE_SHAPES = {"tiny_softmax": dict(T=40, H=256, I=128, E=4, K=2, routing="softmax", seed=11),
                  "tiny_sigmoid_topk4": dict(T=24, H=256, I=128, E=8, K=4, routing="sigmoid", seed=12)}


def write_fixture(path):
    out = {}
    for name, shp in FIXTURE_SHAPES.items():
        for quant in (0, 1, 2, 3):
            c = make_case(quant=quant, **shp)
            n = to_numpy_case(c)
            pre = f"{name}_q{quant}_"
            for k in ("x", "topk_ids", "topk_w", "w1", "w2", "w1_scale", "w2_scale"):
                if n[k] is not None:
                    out[pre + k] = n[k]
            out[pre + "out"] = fused_moe(c).view(torch.int16).numpy().view(np.uint16)
            out[pre + "out_partial_bf16"] = fused_moe(c, partial_bf16=True).view(torch.int16).numpy().view(np.uint16)
    np.savez_compressed(path, **out)
    return out


def load_fixture_case(npz, name, quant):
    pre = f"{name}_q{quant}_"
    d = {k: (npz[pre + k] if pre + k in npz else None)
         for k in ("x", "topk_ids", "topk_w", "w1", "w2", "w1_scale", "w2_scale")}
    d["quant"] = quant
    return d, npz[pre + "out"], npz[pre + "out_partial_bf16"]


if __name__ == "__main__":
    here = os.path.dirname(os.path.abspath(__file__))
    torch.set_num_threads(4)
    write_fixture(os.path.join(here, "torch_ref.npz"))
    print("wrote", os.path.join(here, "torch_ref.npz"), os.path.getsize(os.path.join(here, "torch_ref.npz")), "bytes")
