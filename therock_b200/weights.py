"""Expert weights on disk: one flat file per layer, readable expert by expert.

Layout: 16-byte magic/version, a JSON header (dims, quantisation mode, byte offsets), then the
tensors back to back in exactly the layout the kernels consume -- W1 [E, 2I, H] (gate rows then
up rows), W2 [E, H, I], K contiguous, bf16 or e4m3 bytes, plus f32 scales.  The kernels address
these natural row-major tensors directly through their TMA descriptors; `tile_weights` below is an
optional offline pre-shuffle into contiguous 16 KiB operand tiles (weight_layout = "tiled128":
same results, a faster weight stream for decode-sized batches).  Because experts are the
outermost dimension, an expert-parallel rank maps only its own slice."""
from __future__ import annotations

import json
import os
from typing import Optional

import numpy as np
import torch

MAGIC = b"FMOEW001"


def quantize_experts(w: torch.Tensor, mode: str):
    """[E, rows, cols] float weights -> (stored tensor, scales or None) in the operator's formats:
    "none" -> bf16; "token_channel" -> e4m3 + one scale per output row; "block128" -> e4m3 + one
    scale per 128x128 block.  q = e4m3(w * (1/s)), s = absmax/448 (1 where the group is zero)."""
    if mode == "none":
        return w.to(torch.bfloat16), None
    wf = w.float()
    E, rows, cols = wf.shape
    if mode == "token_channel":
        s = wf.abs().amax(dim=2) / 448.0
        s = torch.where(s > 0, s, torch.ones_like(s))
        q = (wf * (1.0 / s)[:, :, None]).to(torch.float8_e4m3fn).view(torch.uint8)
        return q, s.contiguous()
    if mode == "block128":
        if rows % 128 or cols % 128:
            raise ValueError("block128 needs dimensions that are multiples of 128")
        b = wf.view(E, rows // 128, 128, cols // 128, 128)
        s = b.abs().amax(dim=(2, 4)) / 448.0
        s = torch.where(s > 0, s, torch.ones_like(s))
        q = (b * (1.0 / s)[:, :, None, :, None]).to(torch.float8_e4m3fn).view(torch.uint8).view(E, rows, cols)
        return q, s.contiguous()
    raise ValueError(f"unknown quantisation mode {mode!r}")


def tile_weights(w: torch.Tensor) -> torch.Tensor:
    """Pre-shuffle [E, rows, K] weights (bf16 or e4m3 bytes) into the "tiled128" layout:
    [E, rows/128, K_bytes/128, 128 rows, 128 bytes], i.e. every 128-row x 128-byte operand tile
    becomes one contiguous 16 KiB block.  Returned with the original shape and dtype (the
    bytes are what changes)."""
    E, rows, K = w.shape
    es = w.element_size()
    kt = 128 // es                      # elements per 128 bytes
    if rows % 128 or (K * es) % 128:
        raise ValueError("tiled128 needs rows and K bytes that are multiples of 128")
    t = w.view(E, rows // 128, 128, K // kt, kt).permute(0, 1, 3, 2, 4).contiguous()
    return t.view(E, rows, K)


def untile_weights(w: torch.Tensor) -> torch.Tensor:
    """Inverse of tile_weights."""
    E, rows, K = w.shape
    es = w.element_size()
    kt = 128 // es
    t = w.view(E, rows // 128, K // kt, 128, kt).permute(0, 1, 3, 2, 4).contiguous()
    return t.view(E, rows, K)


def _np(t: torch.Tensor) -> np.ndarray:
    t = t.detach().cpu().contiguous()
    if t.dtype == torch.bfloat16:
        return t.view(torch.int16).numpy().view(np.uint16)
    return t.numpy()


def save_expert_weights(path: str, w1: torch.Tensor, w2: torch.Tensor, quant: str = "none",
                        w1_scale: Optional[torch.Tensor] = None, w2_scale: Optional[torch.Tensor] = None) -> None:
    tensors = {"w1": _np(w1), "w2": _np(w2)}
    if w1_scale is not None:
        tensors["w1_scale"], tensors["w2_scale"] = _np(w1_scale), _np(w2_scale)
    header = {"quant": quant, "E": int(w1.shape[0]), "I": int(w1.shape[1] // 2), "H": int(w1.shape[2]), "tensors": {}}
    off = 0
    for name, a in tensors.items():
        header["tensors"][name] = {"dtype": str(a.dtype), "shape": list(a.shape), "offset": off}
        off += (a.nbytes + 255) // 256 * 256
    hb = json.dumps(header).encode()
    with open(path, "wb") as f:
        f.write(MAGIC + len(hb).to_bytes(8, "little"))
        f.write(hb)
        base = (16 + len(hb) + 255) // 256 * 256
        for name, a in tensors.items():
            f.seek(base + header["tensors"][name]["offset"])
            f.write(a.tobytes())
        f.truncate(base + off)


def load_expert_weights(path: str, device="cpu", experts: Optional[range] = None) -> dict:
    """Returns {"quant", "w1", "w2", "w1_scale", "w2_scale"}; `experts` selects a contiguous
    range (an expert-parallel rank's shard) without reading the rest of the file."""
    with open(path, "rb") as f:
        head = f.read(16)
        if head[:8] != MAGIC:
            raise ValueError(f"{path} is not an expert-weights file")
        hlen = int.from_bytes(head[8:16], "little")
        header = json.loads(f.read(hlen))
    base = (16 + hlen + 255) // 256 * 256
    E = header["E"]
    lo, hi = (0, E) if experts is None else (experts.start, experts.stop)
    if not (0 <= lo <= hi <= E):
        raise ValueError("expert range outside the file")
    out = {"quant": header["quant"], "w1_scale": None, "w2_scale": None}
    for name, meta in header["tensors"].items():
        shape = tuple(meta["shape"])
        mm = np.memmap(path, dtype=np.dtype(meta["dtype"]), mode="r", offset=base + meta["offset"], shape=shape)
        part = np.ascontiguousarray(mm[lo:hi])
        t = torch.from_numpy(part)
        if meta["dtype"] == "uint16":
            t = t.view(torch.bfloat16)
        out[name] = t.to(device)
    return out
