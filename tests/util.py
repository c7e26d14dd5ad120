"""Helpers shared by the GPU parity tests: oracle inputs -> CUDA tensors and back."""
import numpy as np
import torch

from oracle import oracle as O
import therock_b200 as M

QUANT_NAME = {0: "none", 1: "token_channel", 2: "block128", 3: "block128_ue8m0"}


def to_dev(a, dtype=None, device="cuda:0"):
    t = torch.from_numpy(np.ascontiguousarray(a))
    if dtype is not None:
        t = t.view(dtype)
    return t.to(device)


def bf16_dev(bits, device="cuda:0"):
    return to_dev(bits.view(np.int16), torch.bfloat16, device)


def traits_for(quant, partial="f32", gemm_mode=0):
    return M.FusedMoeTraits(prec_w="bf16" if quant == 0 else "fp8", quant=QUANT_NAME[quant], partial_dtype=partial,
                            gemm_mode=gemm_mode)


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


CANARY = 0xA5


def run_gpu(d, partial="f32", gemm_mode=0):
    """One fused_moe call through the C-ABI.  The output and the workspace are allocated with
    64 KiB of canary bytes on either side; the bytes are checked after the run, so a kernel that
    writes outside the buffers it was given fails the test even if the results look right."""
    from therock_b200 import api
    args = args_for(d)
    traits = traits_for(d["quant"], partial, gemm_mode)
    pad = 65536
    T, H = args.a.shape
    need = M.fused_moe_workspace_size(traits, args)
    ws_raw = torch.full((need + 2 * pad + 256,), CANARY, dtype=torch.uint8, device=args.a.device)
    shift = (-(ws_raw.data_ptr() + pad)) % 256
    args.workspace = ws_raw[pad + shift: pad + shift + need]
    out_raw = torch.full((T * H * 2 + 2 * pad,), CANARY, dtype=torch.uint8, device=args.a.device)
    args.o = out_raw[pad: pad + T * H * 2].view(torch.bfloat16).view(T, H)
    out = M.fused_moe(traits, args)
    torch.cuda.synchronize()
    assert api.check_status(args.workspace) == 0
    for name, raw, lo, hi in (("workspace", ws_raw, pad + shift, pad + shift + need),
                              ("output", out_raw, pad, pad + T * H * 2)):
        assert bool((raw[:lo] == CANARY).all()), f"bytes before the {name} were overwritten"
        assert bool((raw[hi:] == CANARY).all()), f"bytes after the {name} were overwritten"
    return out_bits(out), args


def run_oracle(d, sel=None, partial="f32"):
    return O.fused_moe(d["x"], d["w1"], d["w2"], d["topk_ids"], d["topk_w"], d["quant"],
                       d["w1_scale"], d["w2_scale"], sel=sel, partial_bf16=(partial == "bf16"))


def rel_l2(got_bits, ref_bits):
    g, r = O.bf16_to_f32(got_bits), O.bf16_to_f32(ref_bits)
    return float(np.linalg.norm(g - r) / max(np.linalg.norm(r), 1e-30))
