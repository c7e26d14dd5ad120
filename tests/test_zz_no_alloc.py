"""The entry point for callers that cannot allocate device memory (fmoe_run_static_ws).

Such callers -- a plugin slot that is handed only input and output buffers, a foreign
function interface without a CUDA allocator, a loop where cudaMalloc is banned because it
stalls the device -- get the operator's scratch from a 64 MiB array inside the library.
The test calls the entry point through the C-ABI twice in a row and requires the same
bytes as the ordinary entry point with a caller-provided workspace; the second call runs
on top of whatever the first one left in the shared array.  This file is named so that
pytest collects it last."""
import ctypes

import numpy as np
import pytest
import torch

from oracle import oracle as O
import therock_b200 as M
from therock_b200 import api
from tests.util import args_for, out_bits, traits_for

pytestmark = pytest.mark.gpu


def _call_static(traits, args):
    t, a = traits.to_c(), args.to_c()
    rc = api.lib().fmoe_run_static_ws(ctypes.byref(t), ctypes.byref(a), torch.cuda.current_stream().cuda_stream)
    return rc


@pytest.mark.parametrize("quant,shape", [(0, dict(T=128, H=512, I=1024, E=8, K=2)),
                                         (1, dict(T=16, H=1024, I=2048, E=8, K=2))])
def test_static_workspace_matches_caller_workspace_twice(quant, shape):
    d = O.make_inputs(quant=quant, routing="softmax", seed=11, **shape)
    traits = traits_for(quant)
    ref_args = args_for(d)
    ref = M.fused_moe(traits, ref_args)            # ordinary entry point, torch-allocated workspace
    torch.cuda.synchronize()
    assert api.check_status(ref_args.workspace) == 0
    want = out_bits(ref)

    args = args_for(d)
    args.o = torch.empty_like(args.a)
    args.workspace = None                          # nothing is passed: the library's own array is used
    for call in range(2):
        args.o.fill_(float("nan"))
        assert _call_static(traits, args) == 0, api.lib().fmoe_last_error()
        torch.cuda.synchronize()
        got = out_bits(args.o)
        assert (got == want).all(), f"call {call}: differs from fmoe_run"

    # a different problem in between must not disturb the next call (the array is shared)
    d2 = O.make_inputs(T=40, H=256, I=256, E=4, K=2, quant=quant, routing="softmax", seed=12)
    a2 = args_for(d2)
    a2.o = torch.empty_like(a2.a)
    assert _call_static(traits, a2) == 0
    assert _call_static(traits, args) == 0
    torch.cuda.synchronize()
    assert (out_bits(args.o) == want).all()
    ref2 = M.fused_moe(traits, args_for(d2))
    torch.cuda.synchronize()
    assert (out_bits(a2.o) == out_bits(ref2)).all()


def test_static_workspace_rejects_oversized_problems():
    traits = traits_for(0)
    t = traits.to_c()
    a = api._Args()
    a.T, a.H, a.I, a.E, a.K = 4096, 4096, 14336, 8, 2      # needs ~0.5 GB of scratch
    need = ctypes.c_uint64(0)
    assert api.lib().fmoe_get_workspace_size(ctypes.byref(t), ctypes.byref(a), ctypes.byref(need)) == 0
    assert need.value > api.STATIC_WS_BYTES
    rc = api.lib().fmoe_run_static_ws(ctypes.byref(t), ctypes.byref(a), None)
    assert rc == -3
    msg = api.lib().fmoe_last_error().decode()
    assert "built-in workspace" in msg and str(api.STATIC_WS_BYTES) in msg


def test_python_wrapper_requires_the_output_tensor():
    d = O.make_inputs(T=8, H=256, I=128, E=2, K=1, quant=0, routing="softmax", seed=13)
    args = args_for(d)
    with pytest.raises(M.FmoeError):
        api.fused_moe_static_ws(traits_for(0), args)
    args.o = torch.empty_like(args.a)
    out = api.fused_moe_static_ws(traits_for(0), args)
    torch.cuda.synchronize()
    ref = M.fused_moe(traits_for(0), args_for(d))
    torch.cuda.synchronize()
    assert (out_bits(out) == out_bits(ref)).all()
