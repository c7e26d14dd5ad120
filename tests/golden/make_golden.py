"""Generates tests/golden/*.npz.

The reference project holds no source, test or vector for the fused-MoE path, so these
fixtures cannot come from it.  They pin (a) the number-format conversions against an
external implementation (torch's bf16 / float8_e4m3fn casts) and (b) the arithmetic
contract as computed by the *numpy* restatement in oracle/oracle.py, so that the C oracle
and the CUDA path are both checked against something neither of them produced.

Run from the repository root:  python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import oracle as O  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))


def formats():
    import torch
    rng = np.random.default_rng(0)
    x = np.concatenate([
        rng.standard_normal(4096).astype(np.float32) * 3.0,
        rng.standard_normal(2048).astype(np.float32) * 0.01,
        rng.uniform(-448, 448, 2048).astype(np.float32),
        np.array([0.0, -0.0, 448.0, -448.0, 2.0 ** -9, 2.0 ** -10, 1.5 * 2.0 ** -9, 0.0175,
                  2.0 ** -6, 17.0, 18.0, 19.0, 416.0, 432.0, 447.9], np.float32)])
    t = torch.from_numpy(x)
    e4 = t.to(torch.float8_e4m3fn).view(torch.uint8).numpy()
    bf = t.to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)
    table = torch.arange(256, dtype=torch.uint8).view(torch.float8_e4m3fn).float().numpy()
    np.savez_compressed(os.path.join(HERE, "formats.npz"), x=x, e4m3=e4, bf16=bf, e4m3_table=table)


def moe_case(name, T, H, I, E, K, routing, keep_tokens=16):
    logits = O.normal((T, E), 0, 4)
    ids, w = O.np_route(logits, K, routing)
    srt = O.np_moe_sorting(ids, w, E, 128)
    out = dict(logits_head=logits[:8], topk_ids=ids, topk_w=w,
               **{"sort_" + k: v for k, v in srt.items()})
    for quant in (O.QUANT_NONE, O.QUANT_TOKEN_CHANNEL, O.QUANT_BLOCK128):
        d = O.make_inputs(T, H, I, E, K, quant, routing, seed=0)
        assert (d["topk_ids"] == ids).all()
        o = O.np_fused_moe(d["x"], d["w1"], d["w2"], ids, w, quant, d["w1_scale"], d["w2_scale"])
        out[f"out_q{quant}_head"] = o[:keep_tokens]
        out[f"out_q{quant}_sum"] = np.array([O.bf16_to_f32(o).astype(np.float64).sum()])
    np.savez_compressed(os.path.join(HERE, name + ".npz"), **out)


if __name__ == "__main__":
    formats()
    moe_case("c0", **{k: v for k, v in O.CONFIGS["C0"].items() if k != "quant"})
    moe_case("tiny_sigmoid", T=48, H=256, I=256, E=16, K=4, routing="sigmoid")
    print("golden fixtures written to", HERE)
