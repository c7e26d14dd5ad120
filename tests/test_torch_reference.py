"""The C oracle against an independent restatement of the contract in plain torch CPU ops
(tests/golden/torch_reference.py: torch's generator, torch's bf16 / float8_e4m3fn casts,
torch.topk routing, F.linear in float32 -- no helper from oracle/), and against the fixture that
script committed.  Agreement is to float32 round-off: the two sum their dot products in a
different order, so an intermediate value can land on the other side of a bf16 rounding
boundary; the tolerances are the operator's own (bf16 rtol = atol = 1e-2, fp8 relative L2)."""
import os

import numpy as np
import pytest
import torch

from oracle import oracle as O
from tests.golden import torch_reference as TR

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "torch_ref.npz")


def oracle_out(n, partial_bf16=False):
    return O.fused_moe(n["x"], n["w1"], n["w2"], n["topk_ids"], n["topk_w"], n["quant"], n["w1_scale"],
                       n["w2_scale"], partial_bf16=partial_bf16)


def close(got_bits, ref_bits, quant):
    g, r = O.bf16_to_f32(got_bits), O.bf16_to_f32(ref_bits)
    rel = float(np.linalg.norm(g - r) / max(np.linalg.norm(r), 1e-30))
    if quant == 0:
        np.testing.assert_allclose(g, r, rtol=1e-2, atol=1e-2)
    assert rel <= (2e-3 if quant == 0 else 4e-2), rel
    return rel


@pytest.mark.parametrize("quant", [0, 1, 2, 3])
def test_oracle_matches_torch_cpu_on_the_cpu_reference_shape(quant):
    """configs[0] (T=128, H=512, I=1024, E=8, K=2, softmax top-2), inputs drawn by torch."""
    torch.set_num_threads(4)
    c = TR.make_case(128, 512, 1024, 8, 2, quant, "softmax", seed=0)
    ref = TR.fused_moe(c).view(torch.int16).numpy().view(np.uint16)
    rel = close(oracle_out(TR.to_numpy_case(c)), ref, quant)
    assert rel < 5e-3      # far inside the tolerance: only rounding-boundary flips differ


@pytest.mark.parametrize("quant", [2, 3])
def test_oracle_matches_torch_cpu_on_a_down_scaled_fine_grained_shape(quant):
    """The DeepSeek-style configuration scaled down: 64 experts, top-8, sigmoid routing."""
    torch.set_num_threads(4)
    c = TR.make_case(96, 512, 256, 64, 8, quant, "sigmoid", seed=4)
    for partial in (False, True):
        ref = TR.fused_moe(c, partial_bf16=partial).view(torch.int16).numpy().view(np.uint16)
        close(oracle_out(TR.to_numpy_case(c), partial), ref, quant)


def test_routing_matches_torch_topk():
    g = torch.Generator().manual_seed(3)
    logits = torch.randn(257, 40, generator=g)
    for mode in ("softmax", "sigmoid"):
        ids_t, w_t = TR.route(logits, 6, mode)
        ids_o, w_o = O.route(logits.numpy(), 6, mode)
        assert (ids_t.numpy() == ids_o).all()
        np.testing.assert_allclose(w_t.numpy(), w_o, rtol=2e-6, atol=1e-7)


def test_power_of_two_scale_rule_matches_torch():
    a = torch.randn(64, 512, generator=torch.Generator().manual_seed(5)) * torch.logspace(-6, 3, 64)[:, None]
    a[7] = 0.0
    q_t, s_t = TR.quant_groups(a, 128, pow2=True)
    q_o, s_o = O.quant_rows_e4m3(a.numpy(), 128, pow2=True)
    assert (s_t.numpy() == s_o).all()
    assert (np.log2(s_o) == np.round(np.log2(s_o))).all()
    assert (O.e4m3_to_f32(q_o) == q_t.numpy()).all()


@pytest.mark.parametrize("name", sorted(TR.FIXTURE_SHAPES))
@pytest.mark.parametrize("quant", [0, 1, 2, 3])
def test_oracle_matches_the_committed_torch_fixture(name, quant):
    npz = np.load(GOLD)
    d, out, out_pb = TR.load_fixture_case(npz, name, quant)
    close(oracle_out(d), out, quant)
    close(oracle_out(d, True), out_pb, quant)
