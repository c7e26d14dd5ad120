"""`torch.library` binding of the fused operator: `torch.ops.therock_b200.fused_moe`.

The op has a fake (meta) implementation, so it can sit inside traced / compiled graphs, and
its CUDA implementation only enqueues kernels on the current stream (no host sync), so it can
be captured in a CUDA graph.  The workspace comes from torch's caching allocator, which is
graph-pool aware."""
from __future__ import annotations

from typing import Optional

import torch

from . import api


@torch.library.custom_op("therock_b200::fused_moe", mutates_args=(), device_types="cuda")
def fused_moe_op(x: torch.Tensor, w1: torch.Tensor, w2: torch.Tensor, topk_ids: torch.Tensor,
                 topk_weight: torch.Tensor, w1_scale: Optional[torch.Tensor] = None,
                 w2_scale: Optional[torch.Tensor] = None, quant: str = "none") -> torch.Tensor:
    traits = api.FusedMoeTraits(prec_w="bf16" if quant == "none" else "fp8", quant=quant)
    args = api.FusedMoeArgs(a=x, g=w1, d=w2, topk_ids=topk_ids, topk_weight=topk_weight,
                            g_scale=w1_scale, d_scale=w2_scale)
    return api.fused_moe(traits, args)


@fused_moe_op.register_fake
def _(x, w1, w2, topk_ids, topk_weight, w1_scale=None, w2_scale=None, quant="none"):
    return torch.empty_like(x)


@torch.library.custom_op("therock_b200::route", mutates_args=(), device_types="cuda")
def route_op(logits: torch.Tensor, topk: int, mode: str = "softmax") -> tuple[torch.Tensor, torch.Tensor]:
    return api.route(logits, topk, mode)


@route_op.register_fake
def _(logits, topk, mode="softmax"):
    T = logits.shape[0]
    return (torch.empty(T, topk, dtype=torch.int32, device=logits.device),
            torch.empty(T, topk, dtype=torch.float32, device=logits.device))
