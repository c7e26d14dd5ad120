"""Helpers shared by the GPU parity tests: oracle inputs -> CUDA tensors and back."""
import numpy as np
import torch

from oracle import oracle as O
import therock_b200 as M

QUANT_NAME = {0: "none", 1: "token_channel", 2: "block128"}


def to_dev(a, dtype=None, device="cuda:0"):
    t = torch.from_numpy(np.ascontiguousarray(a))
    if dtype is not None:
        t = t.view(dtype)
    return t.to(device)


def bf16_dev(bits, device="cuda:0"):
    return to_dev(bits.view(np.int16), torch.bfloat16, device)


def traits_for(quant):
    return M.FusedMoeTraits(prec_w="bf16" if quant == 0 else "fp8", quant=QUANT_NAME[quant])


def args_for(d, device="cuda:0"):
    q = d["quant"]
    return M.FusedMoeArgs(
        a=bf16_dev(d["x"], device),
        g=bf16_dev(d["w1"], device) if q == 0 else to_dev(d["w1"], device=device),
        d=bf16_dev(d["w2"], device) if q == 0 else to_dev(d["w2"], device=device),
        topk_ids=to_dev(d["topk_ids"], device=device), topk_weight=to_dev(d["topk_w"], device=device),
        g_scale=None if q == 0 else to_dev(d["w1_scale"], device=device),
        d_scale=None if q == 0 else to_dev(d["w2_scale"], device=device))


def out_bits(t):
    return t.view(torch.int16).cpu().numpy().view(np.uint16)


def run_gpu(d):
    args = args_for(d)
    out = M.fused_moe(traits_for(d["quant"]), args)
    torch.cuda.synchronize()
    from therock_b200 import api
    assert api.check_status(args.workspace) == 0
    return out_bits(out), args


def run_oracle(d, sel=None):
    return O.fused_moe(d["x"], d["w1"], d["w2"], d["topk_ids"], d["topk_w"], d["quant"],
                       d["w1_scale"], d["w2_scale"], sel=sel)


def rel_l2(got_bits, ref_bits):
    g, r = O.bf16_to_f32(got_bits), O.bf16_to_f32(ref_bits)
    return float(np.linalg.norm(g - r) / max(np.linalg.norm(r), 1e-30))
