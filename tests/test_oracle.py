"""CPU tests of the oracle: the C restatement against the committed golden fixtures and
against the independent numpy restatement, plus properties of routing and moe_sorting."""
import os

import numpy as np
import pytest

from oracle import oracle as O

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def gold(name):
    return np.load(os.path.join(GOLD, name + ".npz"))


def test_formats_match_torch_fixture():
    g = gold("formats")
    assert (O.f32_to_e4m3(g["x"]) == g["e4m3"]).all()
    assert (O.f32_to_bf16(g["x"]) == g["bf16"]).all()
    tab = O.e4m3_to_f32(np.arange(256, dtype=np.uint8))
    ok = (tab == g["e4m3_table"]) | (np.isnan(tab) & np.isnan(g["e4m3_table"]))
    assert ok.all()
    assert (O.np_f32_to_e4m3(g["x"]) == g["e4m3"]).all()
    assert (O.np_f32_to_bf16(g["x"]) == g["bf16"]).all()


def test_e4m3_saturates_and_rounds_to_even():
    x = np.array([1e9, -1e9, 464.0, 465.0, np.inf, 2.0 ** -10, 3 * 2.0 ** -10, 0.0], np.float32)
    got = O.e4m3_to_f32(O.f32_to_e4m3(x))
    assert got.tolist() == [448.0, -448.0, 448.0, 448.0, 448.0, 0.0, 2 * 2.0 ** -9, 0.0]


def test_quant_rows_scale_and_zero_row():
    a = np.zeros((3, 256), np.float32)
    a[0] = np.linspace(-7, 7, 256)
    a[2, 5] = -3.0
    q, s = O.quant_rows_e4m3(a)
    assert s[:, 0].tolist() == [np.float32(7.0) / np.float32(448.0), 1.0, np.float32(3.0) / np.float32(448.0)]
    assert (q[1] == 0).all() and q[2, 5] == 0xFE
    q2, s2 = O.np_quant(a, 256)
    assert (q == q2).all() and (s == s2).all()
    qg, sg = O.quant_rows_e4m3(a, 128)
    qg2, sg2 = O.np_quant(a, 128)
    assert (qg == qg2).all() and (sg == sg2).all() and sg.shape == (3, 2)


@pytest.mark.parametrize("mode", ["softmax", "sigmoid"])
def test_route_matches_numpy_and_ties_go_low(mode):
    logits = O.normal((257, 19), 3, 4)
    logits[5, :] = 0.25           # full tie: lowest indices win
    logits[6, 3] = logits[6, 11]  # pair tie
    ids, w = O.route(logits, 4, mode)
    ids2, w2 = O.np_route(logits, 4, mode)
    assert (ids == ids2).all()
    np.testing.assert_allclose(w, w2, rtol=1e-6, atol=1e-7)
    assert ids[5].tolist() == [0, 1, 2, 3]
    np.testing.assert_allclose(w.sum(axis=1), 1.0, rtol=1e-6)
    assert all(len(set(r)) == 4 for r in ids.tolist())


@pytest.mark.parametrize("name", ["c0", "tiny_sigmoid"])
def test_sorting_matches_golden(name):
    g = gold(name)
    ids, w = g["topk_ids"], g["topk_w"]
    E = 8 if name == "c0" else 16
    s = O.moe_sorting(ids, w, E, 128)
    for k, v in s.items():
        assert (v == g["sort_" + k]).all(), k


@pytest.mark.parametrize("T,K,E,bm", [(1, 1, 1, 128), (16, 2, 8, 128), (300, 3, 7, 32), (1000, 8, 256, 128),
                                       (64, 2, 8, 1), (0, 2, 4, 128)])
def test_sorting_properties(T, K, E, bm):
    rng = np.random.default_rng(T * 31 + K)
    ids = np.stack([rng.permutation(E)[:K] for _ in range(T)]).astype(np.int32) if T else np.zeros((0, K), np.int32)
    if T > 10:
        ids[3, 0] = -1
        ids[7, K - 1] = E + 5      # out-of-range ids are dropped
    w = rng.random((T, K), dtype=np.float32)
    s = O.moe_sorting(ids, w, E, bm)
    cap = O.sort_capacity(T, K, E, bm)
    npp = int(s["num_tokens_post_pad"][0])
    assert cap % bm == 0 and npp % bm == 0 and npp <= cap
    rows = s["sorted_rows"]
    real = rows[rows >= 0]
    valid = np.nonzero((ids.reshape(-1) >= 0) & (ids.reshape(-1) < E))[0]
    assert sorted(real.tolist()) == valid.tolist()            # every routed pair exactly once
    eids = s["sorted_expert_ids"]
    used = eids[: npp // bm]
    assert (np.diff(used) >= 0).all() and (eids[npp // bm:] == -1).all()
    for b, e in enumerate(used):
        blk = rows[b * bm:(b + 1) * bm]
        r = blk[blk >= 0]
        assert (ids.reshape(-1)[r] == e).all()
        assert (np.diff(r) > 0).all()                          # stable inside the block
        pad = blk < 0
        assert (s["sorted_token_ids"][b * bm:(b + 1) * bm][pad] == T).all()
        assert (s["sorted_weights"][b * bm:(b + 1) * bm][pad] == 0).all()
        assert (s["sorted_token_ids"][b * bm:(b + 1) * bm][~pad] == r // K).all()
    assert (rows[npp:] == -1).all() and (s["sorted_token_ids"][npp:] == T).all()
    cnt = np.bincount(ids.reshape(-1)[valid], minlength=E)
    assert (np.diff(s["mblk_cum"]) == -(-cnt // bm)).all()
    n = O.np_moe_sorting(ids, w, E, bm)
    for k in s:
        assert (s[k] == n[k]).all(), k


@pytest.mark.parametrize("name,cfg", [("c0", O.CONFIGS["C0"]),
                                      ("tiny_sigmoid", dict(T=48, H=256, I=256, E=16, K=4, routing="sigmoid"))])
@pytest.mark.parametrize("quant", [0, 1, 2])
def test_fused_moe_matches_golden(name, cfg, quant):
    g = gold(name)
    c = {k: v for k, v in cfg.items() if k != "quant"}
    d = O.make_inputs(quant=quant, seed=0, **c)
    assert (d["topk_ids"] == g["topk_ids"]).all()
    out = O.fused_moe(d["x"], d["w1"], d["w2"], d["topk_ids"], d["topk_w"], quant, d["w1_scale"], d["w2_scale"])
    head = g[f"out_q{quant}_head"]
    got, ref = O.bf16_to_f32(out[: len(head)]), O.bf16_to_f32(head)
    # two restatements with different summation order: agreement to a bf16 ulp or so
    np.testing.assert_allclose(got, ref, rtol=2e-2, atol=2e-3)
    assert np.linalg.norm(got - ref) / np.linalg.norm(ref) < 2e-3
    assert abs(O.bf16_to_f32(out).astype(np.float64).sum() - float(g[f"out_q{quant}_sum"][0])) < 0.5


def test_fused_moe_token_subset_and_invalid_ids():
    d = O.make_inputs(T=40, H=256, I=128, E=6, K=3, quant=0, seed=1)
    ids = d["topk_ids"].copy()
    ids[4, 1] = -1
    ids[9, :] = 6                       # token with no valid expert -> zero row
    full = O.fused_moe(d["x"], d["w1"], d["w2"], ids, d["topk_w"])
    sel = np.array([9, 4, 39, 0], np.int32)
    part = O.fused_moe(d["x"], d["w1"], d["w2"], ids, d["topk_w"], sel=sel)
    assert (part == full[sel]).all()
    assert (full[9] == 0).all()
    ref = O.np_fused_moe(d["x"], d["w1"], d["w2"], ids, d["topk_w"])
    np.testing.assert_allclose(O.bf16_to_f32(full), O.bf16_to_f32(ref), rtol=2e-2, atol=2e-3)


@pytest.mark.parametrize("quant", [0, 1])
def test_gate_only_oracle_matches_numpy_restatement(quant):
    # W1 is [E, I, H] and y = SiLU(x W1^T): the C oracle against the independent numpy version
    d = O.make_inputs(T=36, H=256, I=256, E=5, K=2, quant=quant, seed=3, gate_only=True)
    assert d["w1"].shape[1] == 256
    out = O.fused_moe(d["x"], d["w1"], d["w2"], d["topk_ids"], d["topk_w"], quant, d["w1_scale"], d["w2_scale"],
                      gate_only=True)
    ref = O.np_fused_moe(d["x"], d["w1"], d["w2"], d["topk_ids"], d["topk_w"], quant, d["w1_scale"],
                         d["w2_scale"], gate_only=True)
    got, want = O.bf16_to_f32(out), O.bf16_to_f32(ref)
    np.testing.assert_allclose(got, want, rtol=2e-2, atol=2e-3)
    assert np.linalg.norm(got - want) / np.linalg.norm(want) < 2e-3


def test_fused_moe_is_linear_in_topk_weight():
    d = O.make_inputs(T=24, H=256, I=128, E=4, K=2, quant=1, seed=2)
    a = O.fused_moe(d["x"], d["w1"], d["w2"], d["topk_ids"], d["topk_w"], 1, d["w1_scale"], d["w2_scale"])
    b = O.fused_moe(d["x"], d["w1"], d["w2"], d["topk_ids"], d["topk_w"] * np.float32(4.0), 1, d["w1_scale"], d["w2_scale"])
    assert (O.bf16_to_f32(b) == 4.0 * O.bf16_to_f32(a)).all()     # power-of-two scaling is exact


def test_philox_generator_is_index_addressed():
    a = O.normal((1000,), 7, 2)
    b = O.normal((250, 4), 7, 2)
    assert (a == b.reshape(-1)).all()
    assert abs(float(O.normal((200000,), 0, 1).std()) - 1.0) < 0.01
