"""GPU parity tests: the CUDA path, called through the C-ABI, against the CPU oracle.

Tolerances (from the task statement): moe_sorting bit-exact; bf16 rtol = atol = 1e-2;
fp8 relative L2 <= 4e-2."""
import os

import numpy as np
import pytest
import torch

from oracle import oracle as O
import therock_b200 as M
from therock_b200 import api
from tests.util import (QUANT_NAME, args_for, bf16_dev, out_bits, rel_l2, run_gpu, run_oracle, to_dev, traits_for)

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
BF16_TOL = dict(rtol=1e-2, atol=1e-2)
FP8_REL_L2 = 4e-2


def check(d, got, ref):
    g, r = O.bf16_to_f32(got), O.bf16_to_f32(ref)
    assert not np.isnan(g).any()
    if d["quant"] == 0:
        np.testing.assert_allclose(g, r, **BF16_TOL)
    assert rel_l2(got, ref) <= (2e-3 if d["quant"] == 0 else FP8_REL_L2)


# ------------------------------------------------------------------------------ moe_sorting

SORT_CASES = [(128, 2, 8, "softmax"), (4096, 2, 8, "softmax"), (8192, 2, 8, "softmax"), (16, 2, 8, "softmax"),
              (8192, 8, 256, "sigmoid"), (1, 1, 1, "softmax"), (3, 5, 5, "softmax"), (777, 3, 17, "softmax"),
              (33, 1, 300, "sigmoid")]


@pytest.mark.parametrize("T,K,E,mode", SORT_CASES)
def test_moe_sorting_bit_exact(T, K, E, mode):
    ids, w = O.route(O.normal((T, E), 0, 4), K, mode)
    if T >= 100:
        ids[::7, 0] = -1
        ids[::11, K - 1] = E + 3
    ref = O.moe_sorting(ids, w, E, 128)
    got = M.moe_sorting(to_dev(ids), to_dev(w), E, 128)
    torch.cuda.synchronize()
    assert (got[0].cpu().numpy() == ref["sorted_token_ids"]).all()
    assert (got[1].cpu().numpy().view(np.uint32) == ref["sorted_weights"].view(np.uint32)).all()
    assert (got[2].cpu().numpy() == ref["sorted_expert_ids"]).all()
    assert int(got[3].item()) == int(ref["num_tokens_post_pad"][0])


@pytest.mark.parametrize("bm", [1, 16, 32, 64, 256])
def test_moe_sorting_other_block_sizes(bm):
    ids, w = O.route(O.normal((500, 12), 1, 4), 3, "softmax")
    ref = O.moe_sorting(ids, w, 12, bm)
    got = M.moe_sorting(to_dev(ids), to_dev(w), 12, bm)
    torch.cuda.synchronize()
    assert (got[0].cpu().numpy() == ref["sorted_token_ids"]).all()
    assert (got[2].cpu().numpy() == ref["sorted_expert_ids"]).all()
    assert int(got[3].item()) == int(ref["num_tokens_post_pad"][0])


def test_moe_sorting_skewed_and_all_one_expert():
    T, K, E = 2000, 2, 8
    ids = np.zeros((T, K), np.int32)
    ids[:, 1] = 5                                   # only experts 0 and 5 are hit
    w = np.full((T, K), 0.5, np.float32)
    ref = O.moe_sorting(ids, w, E, 128)
    got = M.moe_sorting(to_dev(ids), to_dev(w), E, 128)
    torch.cuda.synchronize()
    assert (got[0].cpu().numpy() == ref["sorted_token_ids"]).all()
    assert (got[2].cpu().numpy() == ref["sorted_expert_ids"]).all()


def test_sort_stage_inside_fused_moe_is_bit_exact():
    d = O.make_inputs(**O.CONFIGS["C0"])
    _, args = run_gpu(d)
    lay = M.workspace_layout(traits_for(0), args)
    ref = O.moe_sorting(d["topk_ids"], d["topk_w"], 8, 128)
    ws = args.workspace
    cap = lay["capacity"]

    def region(name, n, dt):
        return ws[lay[name]:lay[name] + 4 * n].view(dt).cpu().numpy()
    assert (region("sorted_token_ids", cap, torch.int32) == ref["sorted_token_ids"]).all()
    assert (region("sorted_rows", cap, torch.int32) == ref["sorted_rows"]).all()
    assert (region("sorted_weights", cap, torch.int32) == ref["sorted_weights"].view(np.int32)).all()
    assert (region("sorted_expert_ids", cap // 128, torch.int32) == ref["sorted_expert_ids"]).all()
    assert (region("mblk_cum", 9, torch.int32) == ref["mblk_cum"]).all()
    assert int(region("meta", 2, torch.int32)[0]) == int(ref["num_tokens_post_pad"][0])


@pytest.mark.parametrize("T,K,E,quant", [(16, 2, 8, 1), (16, 2, 8, 0), (40, 3, 300, 1), (1, 1, 1, 0), (128, 1, 5, 1),
                                          (9, 8, 256, 0)])
def test_decode_prologue_sorting_is_bit_exact(T, K, E, quant):
    """Decode-sized batches (at most 128 routed pairs) run moe_sorting and the gather as one
    kernel: its sorted arrays must be the oracle's, bit for bit, invalid ids included."""
    H, I = 256, 128
    d = O.make_inputs(T, H, I, E, K, quant, "sigmoid", seed=T + E)
    if T > 4:
        d["topk_ids"][1, 0] = -1
        d["topk_ids"][3, K - 1] = E + 2
    got, args = run_gpu(d)
    lay = M.workspace_layout(traits_for(quant), args)
    ref = O.moe_sorting(d["topk_ids"], d["topk_w"], E, 128)
    ws, cap = args.workspace, lay["capacity"]

    def region(name, n):
        return ws[lay[name]:lay[name] + 4 * n].view(torch.int32).cpu().numpy()
    assert (region("sorted_token_ids", cap) == ref["sorted_token_ids"]).all()
    assert (region("sorted_rows", cap) == ref["sorted_rows"]).all()
    assert (region("sorted_weights", cap) == ref["sorted_weights"].view(np.int32)).all()
    assert (region("sorted_expert_ids", cap // 128) == ref["sorted_expert_ids"]).all()
    assert (region("mblk_cum", E + 1) == ref["mblk_cum"]).all()
    assert int(region("meta", 2)[0]) == int(ref["num_tokens_post_pad"][0])
    check(d, got, run_oracle(d))


# ------------------------------------------------------------------------------ fused MoE

@pytest.mark.parametrize("quant", [0, 1, 2, 3])
def test_c0_matches_oracle_and_golden(quant):
    d = O.make_inputs(**{**O.CONFIGS["C0"], "quant": quant})
    got, _ = run_gpu(d)
    check(d, got, run_oracle(d))
    if quant == 3:
        return          # the fixture file holds the three f32-scale modes
    g = np.load(os.path.join(GOLD, "c0.npz"))
    head = g[f"out_q{quant}_head"]
    check(d, got[: len(head)], head)


@pytest.mark.parametrize("quant", [0, 1, 2, 3])
@pytest.mark.parametrize("T,H,I,E,K", [(1, 256, 128, 1, 1), (77, 256, 384, 5, 3), (16, 1024, 2048, 8, 2),
                                       (300, 512, 256, 16, 4), (129, 768, 640, 3, 2)])
def test_ragged_shapes(quant, T, H, I, E, K):
    d = O.make_inputs(T, H, I, E, K, quant, "softmax", seed=T)
    got, _ = run_gpu(d)
    check(d, got, run_oracle(d))


@pytest.mark.parametrize("quant", [0, 1, 2, 3])
def test_invalid_expert_ids_are_skipped(quant):
    d = O.make_inputs(64, 256, 256, 6, 3, quant, "softmax", seed=5)
    d["topk_ids"][4, 1] = -1
    d["topk_ids"][9, :] = 6
    d["topk_ids"][10, 0] = 1000
    got, _ = run_gpu(d)
    check(d, got, run_oracle(d))
    assert (got[9] == 0).all()


def test_empty_experts_and_skew():
    d = O.make_inputs(512, 256, 256, 8, 2, 0, "softmax", seed=6)
    d["topk_ids"][:, 0] = 2
    d["topk_ids"][:, 1] = 7
    got, _ = run_gpu(d)
    check(d, got, run_oracle(d))


@pytest.mark.parametrize("partial", ["f32", "bf16"])
@pytest.mark.parametrize("T,H,I,E,K", [(200, 1792, 256, 6, 2), (64, 3584, 128, 3, 1)])
def test_hardware_scaled_down_gemm_with_224_column_tiles(T, H, I, E, K, partial):
    """Hidden sizes that are multiples of 224 (as 7168 is) run the second GEMM of the UE8M0 mode
    with two 224-column accumulators in tensor memory; the tile's 32-row scale groups then cut
    across the 128-row weight-scale blocks."""
    d = O.make_inputs(T, H, I, E, K, 3, "softmax", seed=H + T)
    got, _ = run_gpu(d, partial, gemm_mode=1)      # tokens on M: the kernel with the 224-column tiles
    check(d, got, run_oracle(d, partial=partial))


@pytest.mark.parametrize("quant", [1, 2, 3])
@pytest.mark.parametrize("T,H,I,E,K", [(200, 512, 256, 8, 2), (77, 256, 384, 5, 1), (16, 1024, 128, 8, 2)])
def test_prequantised_activations_give_identical_bits(quant, T, H, I, E, K):
    """Activations quantised by fmoe_quantise_rows and passed as e4m3 rows + scales (what the
    receiving side of an e4m3 expert-parallel dispatch does) give the bits of the bf16 call."""
    d = O.make_inputs(T, H, I, E, K, quant, "softmax", seed=7 * T + quant)
    ref, _ = run_gpu(d)
    args = args_for(d)
    q, s = api.quantise_rows(args.a, QUANT_NAME[quant])
    args.a, args.a_scale = q, s
    got = out_bits(M.fused_moe(traits_for(quant), args))
    torch.cuda.synchronize()
    assert api.check_status(args.workspace) == 0
    assert (got == ref).all()
    # the stand-alone quantisation against the oracle's, bit for bit (bytes and scales)
    q_ref, s_ref = O.quant_rows_e4m3(O.bf16_to_f32(d["x"]), None if quant == 1 else 128, pow2=(quant == 3))
    assert (q.cpu().numpy() == q_ref).all()
    if quant == 3:
        s_got = s.cpu().numpy()[:, :H // 128]
        assert (s_got == ((s_ref.view(np.uint32) >> 23) & 0xff).astype(np.uint8)).all()
    else:
        assert (s.cpu().numpy().view(np.float32).reshape(s_ref.shape) == s_ref).all()


TOKENS_ON_N_CASES = [
    (300, 512, 384, 6, 2, "spread"),      # ~100 rows per expert: one chunk each
    (1500, 512, 256, 4, 2, "spread"),     # ~750 rows per expert: four chunks of unequal size
    (40, 256, 128, 16, 1, "spread"),      # most experts hold 0..5 rows, some none
    (700, 1792, 256, 3, 1, "spread"),     # ~233 rows per expert: around the 224-token chunk limit
    (1024, 256, 256, 8, 1, "one"),        # every row on one expert: five chunks, seven experts empty
    (449, 256, 128, 2, 1, "one"),         # 449 rows: three chunks of 160 + 144 + 160 after rounding to 464
]


@pytest.mark.parametrize("partial", ["f32", "bf16"])
@pytest.mark.parametrize("T,H,I,E,K,routing", TOKENS_ON_N_CASES)
def test_ue8m0_tokens_on_n_kernel_matches_oracle_and_tokens_on_m(T, H, I, E, K, routing, partial):
    """The UE8M0 mode has two GEMM kernels: tokens as 128-row blocks on M, or weights on M and an
    expert's live tokens, in steps of 16, on N.  Both are checked against the oracle on ragged
    expert loads and against each other (same products, same K order: the results agree to well
    inside one bf16 rounding of the output)."""
    d = O.make_inputs(T, H, I, E, K, 3, "softmax", seed=3 * T + E)
    if routing == "one":
        d["topk_ids"][:] = E - 1
    ref = run_oracle(d, partial=partial)
    on_n, _ = run_gpu(d, partial, gemm_mode=2)
    check(d, on_n, ref)
    on_m, _ = run_gpu(d, partial, gemm_mode=1)
    check(d, on_m, ref)
    assert rel_l2(on_n, on_m) <= 2e-3


@pytest.mark.parametrize("quant", [0, 1, 3])
def test_shared_expert_as_one_more_expert_every_token_selects(quant):
    """A DeepSeek-style shared expert in the same call: expert E-1 holds its weights and
    append_shared_expert gives every token one more (expert, weight 1) pair."""
    T, H, I, E, K = 160, 512, 256, 9, 2
    d = O.make_inputs(T, H, I, E, K, quant, "sigmoid", seed=77)
    d["topk_ids"] = np.where(d["topk_ids"] == E - 1, (d["topk_ids"] + 1) % (E - 1), d["topk_ids"]).astype(np.int32)
    ids, w = api.append_shared_expert(to_dev(d["topk_ids"]), to_dev(d["topk_w"]), E - 1)
    d2 = dict(d, topk_ids=ids.cpu().numpy(), topk_w=w.cpu().numpy())
    assert d2["topk_ids"].shape == (T, K + 1) and (d2["topk_ids"][:, K] == E - 1).all()
    got, _ = run_gpu(d2)
    check(d2, got, run_oracle(d2))


def test_tiny_sigmoid_golden():
    cfg = dict(T=48, H=256, I=256, E=16, K=4, routing="sigmoid")
    g = np.load(os.path.join(GOLD, "tiny_sigmoid.npz"))
    for quant in (0, 1, 2):
        d = O.make_inputs(quant=quant, **cfg)
        got, _ = run_gpu(d)
        check(d, got[:16], g[f"out_q{quant}_head"])


@pytest.mark.parametrize("quant", [0, 1, 2, 3])
@pytest.mark.parametrize("T,H,I,E,K", [(200, 512, 256, 8, 2), (77, 256, 384, 5, 3)])
def test_bf16_partial_rows_match_their_oracle_mode(quant, T, H, I, E, K):
    """partial_dtype = bf16: every weighted expert output is rounded to bf16 before the ordered
    sum.  Checked against the oracle mode that does exactly that, at the normal tolerance."""
    d = O.make_inputs(T, H, I, E, K, quant, "softmax", seed=T + quant)
    got, _ = run_gpu(d, partial="bf16")
    check(d, got, run_oracle(d, partial="bf16"))


def test_zero_tokens_is_a_no_op():
    d = O.make_inputs(4, 256, 128, 2, 1, 0, "softmax", seed=7)
    args = args_for(d)
    args.a = args.a[:0].contiguous()
    args.topk_ids = args.topk_ids[:0].contiguous()
    args.topk_weight = args.topk_weight[:0].contiguous()
    out = M.fused_moe(traits_for(0), args)
    torch.cuda.synchronize()
    assert out.shape == (0, 256)


# ------------------------------------------------------------------------------ properties

@pytest.mark.parametrize("quant", [0, 1, 2, 3])
def test_linear_in_topk_weight_bit_exact(quant):
    d = O.make_inputs(200, 512, 256, 8, 2, quant, "softmax", seed=8)
    a, _ = run_gpu(d)
    d2 = dict(d)
    d2["topk_w"] = d["topk_w"] * np.float32(0.25)
    b, _ = run_gpu(d2)
    assert (O.bf16_to_f32(b) == 0.25 * O.bf16_to_f32(a)).all()


@pytest.mark.parametrize("quant", [0, 1, 2, 3])
def test_token_permutation_permutes_output_bit_exact(quant):
    d = O.make_inputs(300, 256, 256, 8, 2, quant, "softmax", seed=9)
    a, _ = run_gpu(d)
    perm = np.random.default_rng(0).permutation(300)
    d2 = dict(d)
    for k in ("x", "topk_ids", "topk_w"):
        d2[k] = np.ascontiguousarray(d[k][perm])
    b, _ = run_gpu(d2)
    assert (b == a[perm]).all()


def test_repeat_runs_are_deterministic():
    d = O.make_inputs(500, 512, 512, 8, 2, 0, "softmax", seed=10)
    a, _ = run_gpu(d)
    for _ in range(3):
        b, _ = run_gpu(d)
        assert (a == b).all()


# ------------------------------------------------------------------------------ full-size configurations

def _coverage_tokens(sorted_tok, npp, mblk_cum, T, n_blocks_wanted, rng):
    """Tokens that cover every expert that received rows and the first and the last live slot
    of at least `n_blocks_wanted` row blocks (all of them when there are fewer), plus a few
    random tokens."""
    n_blocks = npp // 128
    blocks = np.arange(n_blocks)
    if n_blocks > n_blocks_wanted:
        # every expert's first and last block, then evenly spread ones
        edges = np.unique(np.concatenate([mblk_cum[:-1][np.diff(mblk_cum) > 0], mblk_cum[1:][np.diff(mblk_cum) > 0] - 1]))
        rest = rng.choice(n_blocks, size=n_blocks_wanted, replace=False)
        blocks = np.unique(np.concatenate([edges, rest]))
    sel = []
    for b in blocks:
        seg = sorted_tok[b * 128:(b + 1) * 128]
        live = np.nonzero(seg < T)[0]
        if len(live):
            sel += [int(seg[live[0]]), int(seg[live[-1]])]
    sel += rng.choice(T, size=min(8, T), replace=False).tolist()
    return np.unique(np.array(sel, dtype=np.int32))


def _full_size(name, n_blocks_wanted=64, gemm_mode=0):
    """Inputs generated on the device at the configuration's full size (the benchmark's own
    generator).  The oracle evaluates the tokens that sit in the first and the last live slot of
    at least 64 row blocks -- every expert's first and last block among them -- so every expert
    and the block boundaries of the tile schedule are looked at (each token's output depends only
    on its own row)."""
    import bench
    c = bench.CONFIGS[name]
    quant, T, E = c["quant"], c["T"], c["E"]
    d = bench.device_inputs(c, torch.device("cuda:0"))
    args = M.FusedMoeArgs(a=d["x"], g=d["w1"], d=d["w2"], topk_ids=d["ids"], topk_weight=d["w"],
                          g_scale=d["s1"], d_scale=d["s2"])
    out = M.fused_moe(traits_for(quant, gemm_mode=gemm_mode), args)
    torch.cuda.synchronize()
    assert api.check_status(args.workspace) == 0
    lay = M.workspace_layout(traits_for(quant, gemm_mode=gemm_mode), args)
    ws, cap = args.workspace, lay["capacity"]
    tok = ws[lay["sorted_token_ids"]:lay["sorted_token_ids"] + 4 * cap].view(torch.int32).cpu().numpy()
    cum = ws[lay["mblk_cum"]:lay["mblk_cum"] + 4 * (E + 1)].view(torch.int32).cpu().numpy()
    npp = int(ws[lay["meta"]:lay["meta"] + 4].view(torch.int32).item())
    sel = (np.arange(T, dtype=np.int32) if T <= 64 else
           _coverage_tokens(tok, npp, cum, T, n_blocks_wanted, np.random.default_rng(1)))
    ids_h = d["ids"].cpu().numpy()
    hit = np.unique(ids_h[sel])
    assert set(hit.tolist()) == set(np.unique(ids_h).tolist()), "every expert with rows is covered"
    w1 = out_bits(d["w1"]) if quant == 0 else d["w1"].cpu().numpy()
    w2 = out_bits(d["w2"]) if quant == 0 else d["w2"].cpu().numpy()
    ref = O.fused_moe(out_bits(d["x"]), w1, w2, ids_h, d["w"].cpu().numpy(), quant,
                      None if d["s1"] is None else d["s1"].cpu().numpy(),
                      None if d["s2"] is None else d["s2"].cpu().numpy(), sel=sel)
    check(dict(quant=quant), out_bits(out)[sel], ref)
    return len(sel)


def test_full_size_mixtral_prefill_bf16():
    assert _full_size("C1") >= 128


def test_full_size_mixtral_prefill_fp8():
    assert _full_size("C2") >= 128


def test_full_size_decode_fp8():
    assert _full_size("C3") == 16


def test_full_size_deepseek_block_scaled_fp8():
    assert _full_size("C4", n_blocks_wanted=256) >= 512


def test_full_size_deepseek_block_scaled_fp8_power_of_two_scales():
    assert _full_size("C4m", n_blocks_wanted=256) >= 512


def test_full_size_deepseek_power_of_two_scales_tokens_on_n_kernel():
    """The selectable kernel form (weights on M, tokens on N) at the full DeepSeek-V3-shape size:
    256 experts with 200-320 live rows each, i.e. two chunks of unequal size per expert."""
    assert _full_size("C4m", n_blocks_wanted=128, gemm_mode=2) >= 256


def test_deepseek_shape_block_scaled_reduced():
    """The fine-grained configuration (256 experts, top-8, sigmoid routing, 1x128 / 128x128
    scales) at a reduced token count and expert width that the oracle finishes in seconds."""
    d = O.make_inputs(512, 1024, 256, 256, 8, 2, "sigmoid", seed=3)
    got, _ = run_gpu(d)
    check(d, got, run_oracle(d))


# ------------------------------------------------------------------------------ router

@pytest.mark.parametrize("T,E,K,mode", [(128, 8, 2, "softmax"), (4096, 8, 2, "softmax"), (8192, 256, 8, "sigmoid"),
                                        (33, 300, 5, "softmax"), (7, 17, 17, "sigmoid"), (1, 1, 1, "softmax")])
def test_router_matches_oracle(T, E, K, mode):
    logits = O.normal((T, E), 5, 4)
    if T > 4:
        logits[3, :] = 0.5                      # full tie: the K lowest indices win
        logits[2, E - 1] = logits[2, 0]
    ref_ids, ref_w = O.route(logits, K, mode)
    ids, w = M.route(to_dev(logits), K, mode)
    torch.cuda.synchronize()
    ids, w = ids.cpu().numpy(), w.cpu().numpy()
    same = ids == ref_ids
    if not same.all():
        # a different pick is only acceptable between scores that are equal to rounding
        s = logits if mode == "sigmoid" else logits - logits.max(axis=1, keepdims=True)
        t_idx, k_idx = np.nonzero(~same)
        assert np.abs(s[t_idx, ids[t_idx, k_idx]] - s[t_idx, ref_ids[t_idx, k_idx]]).max() < 1e-5
        assert (~same).mean() < 1e-3
    np.testing.assert_allclose(w[same], ref_w[same], rtol=2e-6, atol=1e-7)
    if T > 4:
        assert ids[3].tolist() == list(range(K))
    np.testing.assert_allclose(w.sum(axis=1), 1.0, rtol=1e-5)


def test_router_feeds_fused_moe():
    d = O.make_inputs(**O.CONFIGS["C0"])
    ids, w = M.route(to_dev(d["logits"]), 2, "softmax")
    args = args_for(d)
    args.topk_ids, args.topk_weight = ids, w
    out = M.fused_moe(traits_for(0), args)
    torch.cuda.synchronize()
    d2 = dict(d)
    d2["topk_ids"], d2["topk_w"] = ids.cpu().numpy(), w.cpu().numpy()
    check(d2, out_bits(out), run_oracle(d2))


# ------------------------------------------------------------------------------ graph capture / torch op

@pytest.mark.parametrize("quant", [0, 1])
def test_cuda_graph_replay_matches_eager(quant):
    d = O.make_inputs(64, 512, 512, 8, 2, quant, "softmax", seed=31)
    args = args_for(d)
    args.o = torch.empty_like(args.a)
    args.workspace = torch.empty(M.fused_moe_workspace_size(traits_for(quant), args), dtype=torch.uint8, device="cuda:0")
    eager = out_bits(M.fused_moe(traits_for(quant), args)).copy()
    torch.cuda.synchronize()
    side = torch.cuda.Stream()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        M.fused_moe(traits_for(quant), args)            # warm-up on the capture stream
        side.synchronize()
        with torch.cuda.graph(graph, stream=side):
            M.fused_moe(traits_for(quant), args)
    for _ in range(3):
        args.o.zero_()
        graph.replay()
        torch.cuda.synchronize()
        assert (out_bits(args.o) == eager).all()
    assert api.check_status(args.workspace) == 0


def test_torch_library_op():
    import therock_b200.torch_op  # noqa: F401  (registers torch.ops.therock_b200.*)
    d = O.make_inputs(40, 256, 256, 4, 2, 1, "softmax", seed=32)
    a = args_for(d)
    ids, w = torch.ops.therock_b200.route(to_dev(d["logits"]), 2, "softmax")
    out = torch.ops.therock_b200.fused_moe(a.a, a.g, a.d, ids, w, a.g_scale, a.d_scale, "token_channel")
    torch.cuda.synchronize()
    d2 = dict(d)
    d2["topk_ids"], d2["topk_w"] = ids.cpu().numpy(), w.cpu().numpy()
    check(d2, out_bits(out), run_oracle(d2))
    # fake (meta) implementation: shape inference without running the kernels
    from torch._subclasses.fake_tensor import FakeTensorMode
    with FakeTensorMode():
        fx = torch.empty(40, 256, dtype=torch.bfloat16, device="cuda")
        fo = torch.ops.therock_b200.fused_moe(fx, torch.empty(4, 512, 256, dtype=torch.uint8, device="cuda"),
                                              torch.empty(4, 256, 256, dtype=torch.uint8, device="cuda"),
                                              torch.empty(40, 2, dtype=torch.int32, device="cuda"),
                                              torch.empty(40, 2, device="cuda"), None, None, "token_channel")
        assert fo.shape == (40, 256) and fo.dtype == torch.bfloat16


def test_random_small_configurations():
    """Seeded sweep over ragged shapes and all three quantisation modes."""
    rng = np.random.default_rng(2024)
    for case in range(14):
        T = int(rng.integers(1, 300))
        H = int(rng.choice([256, 512, 768]))
        I = int(rng.choice([128, 256, 384]))
        E = int(rng.integers(1, 13))
        K = int(rng.integers(1, min(E, 4) + 1))
        quant = int(rng.integers(0, 4))
        d = O.make_inputs(T, H, I, E, K, quant, "softmax" if case % 2 else "sigmoid", seed=100 + case)
        if T > 5:
            d["topk_ids"][int(rng.integers(0, T)), 0] = -1
        got, _ = run_gpu(d)
        check(d, got, run_oracle(d))


# ------------------------------------------------------------------------------ C++ host surface

@pytest.mark.parametrize("quant", [0, 1])
def test_cpp_host_program_through_fused_moe_hpp(quant, tmp_path):
    """Builds tests/cpp/fused_moe_cpp_host.cpp (fused_moe_traits / fused_moe_args /
    fused_moe(traits, args, stream) and moe_sorting from include/fused_moe.hpp) with nvcc,
    links it against libfmoe_b200.so, runs it on one problem and checks its outputs."""
    import subprocess
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    exe = str(tmp_path / "fmoe_cpp_host")
    libdir = os.path.join(root, "therock_b200")
    env = {k: v for k, v in os.environ.items() if k not in ("CC", "CXX")}
    subprocess.run(["nvcc", "-std=c++17", "-O2", "-I", os.path.join(root, "include"), "-o", exe,
                    os.path.join(root, "tests", "cpp", "fused_moe_cpp_host.cpp"), "-L", libdir,
                    "-l:libfmoe_b200.so", "-Xlinker", "-rpath", "-Xlinker", libdir], check=True, env=env)
    T, H, I, E, K = 96, 512, 256, 8, 2
    d = O.make_inputs(T, H, I, E, K, quant, "softmax", seed=41)
    prob, res = str(tmp_path / "problem.bin"), str(tmp_path / "result.bin")
    with open(prob, "wb") as f:
        f.write(np.array([T, H, I, E, K, quant], np.int32).tobytes())
        for name in ("x", "w1", "w2"):
            f.write(np.ascontiguousarray(d[name]).tobytes())
        if quant:
            f.write(d["w1_scale"].astype(np.float32).tobytes())
            f.write(d["w2_scale"].astype(np.float32).tobytes())
        f.write(d["topk_ids"].astype(np.int32).tobytes())
        f.write(d["topk_w"].astype(np.float32).tobytes())
    r = subprocess.run([exe, prob, res], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr + r.stdout
    raw = open(res, "rb").read()
    cap = O.sort_capacity(T, K, E, 128)
    npp = int(np.frombuffer(raw[:4], np.int32)[0])
    sids = np.frombuffer(raw[4:4 + cap * 4], np.int32)
    out = np.frombuffer(raw[4 + cap * 4:], np.uint16).reshape(T, H)
    ref_sort = O.moe_sorting(d["topk_ids"], d["topk_w"], E, 128)
    assert npp == int(ref_sort["num_tokens_post_pad"][0]) and (sids == ref_sort["sorted_token_ids"]).all()
    check(d, out, run_oracle(d))


@pytest.mark.parametrize("quant", [0, 1, 2, 3])
@pytest.mark.parametrize("gemm_mode", [1, 2])
def test_tiled_weight_layout_gives_identical_results(quant, gemm_mode):
    from therock_b200 import weights as W
    d = O.make_inputs(300, 512, 384, 6, 2, quant, "softmax", seed=51)
    base = args_for(d)
    tr = traits_for(quant)
    tr.gemm_mode = gemm_mode
    ref = out_bits(M.fused_moe(tr, base)).copy()
    tiled = args_for(d)
    tiled.g, tiled.d = W.tile_weights(tiled.g), W.tile_weights(tiled.d)
    tr2 = traits_for(quant)
    tr2.gemm_mode = gemm_mode
    tr2.weight_layout = "tiled128"
    got = out_bits(M.fused_moe(tr2, tiled))
    torch.cuda.synchronize()
    assert (got == ref).all()
    check(d, got, run_oracle(d))


@pytest.mark.parametrize("T,K,E", [(8192, 8, 256), (5000, 2, 8), (4096, 2, 8), (20000, 3, 1000), (8192, 1, 1)])
def test_multi_cta_sorting_inside_fused_moe_is_bit_exact(T, K, E):
    """fmoe_run uses the multi-CTA moe_sorting for >= 8192 pairs: same bits as the oracle."""
    ids, w = O.route(O.normal((T, E), 7, 4), K, "softmax")
    ids[::9, 0] = -1
    H, I = 256, 128
    d = dict(x=O.f32_to_bf16(O.normal((T, H), 7, 1)), w1=O.f32_to_bf16(O.normal((E, 2 * I, H), 7, 2, 0.02)),
             w2=O.f32_to_bf16(O.normal((E, H, I), 7, 3, 0.02)), topk_ids=ids, topk_w=w, quant=0, w1_scale=None,
             w2_scale=None)
    args = args_for(d)
    M.fused_moe(traits_for(0), args)
    torch.cuda.synchronize()
    lay = M.workspace_layout(traits_for(0), args)
    ref = O.moe_sorting(ids, w, E, 128)
    ws, cap = args.workspace, lay["capacity"]

    def region(name, n):
        return ws[lay[name]:lay[name] + 4 * n].view(torch.int32).cpu().numpy()
    assert (region("sorted_token_ids", cap) == ref["sorted_token_ids"]).all()
    assert (region("sorted_rows", cap) == ref["sorted_rows"]).all()
    assert (region("sorted_weights", cap) == ref["sorted_weights"].view(np.int32)).all()
    assert (region("sorted_expert_ids", cap // 128) == ref["sorted_expert_ids"]).all()
    assert (region("mblk_cum", E + 1) == ref["mblk_cum"]).all()
    assert int(region("meta", 2)[0]) == int(ref["num_tokens_post_pad"][0])


def test_host_pipeline_overlaps_copies_and_keeps_results():
    """Host-resident batches through HostPipeline: every batch is copied in, computed and
    copied back; different batches must not disturb each other although their copies overlap."""
    d = O.make_inputs(128, 512, 256, 8, 2, 0, "softmax", seed=61)
    args = args_for(d)
    traits = traits_for(0)
    args.workspace = torch.empty(M.fused_moe_workspace_size(traits, args), dtype=torch.uint8, device="cuda:0")
    outs = [torch.empty_like(args.a) for _ in range(2)]

    def step(x, ids, w, slot):
        args.a, args.topk_ids, args.topk_weight, args.o = x, ids, w, outs[slot]
        return M.fused_moe(traits, args)
    pipe = api.HostPipeline(step, 128, 512, 2, torch.device("cuda:0"), depth=2)
    n = 6
    xs = [torch.from_numpy(O.f32_to_bf16(O.normal((128, 512), 70 + i, 1)).view(np.int16)).view(torch.bfloat16).pin_memory()
          for i in range(n)]
    ids_h = torch.from_numpy(d["topk_ids"]).pin_memory()
    w_h = torch.from_numpy(d["topk_w"]).pin_memory()
    res = [torch.empty(128, 512, dtype=torch.bfloat16).pin_memory() for _ in range(n)]
    for i in range(n):
        pipe.submit(xs[i], ids_h, w_h, res[i])
    pipe.drain()
    for i in range(n):
        di = dict(d)
        di["x"] = xs[i].view(torch.int16).numpy().view(np.uint16)
        check(di, res[i].view(torch.int16).numpy().view(np.uint16), run_oracle(di))


def test_graph_pipeline_one_launch_per_step_keeps_results():
    """GraphPipeline: the step, the copy-in of the next batch and the copy-out of the previous
    result run as branches of one CUDA graph per step; every batch must still get its own result."""
    d = O.make_inputs(128, 512, 256, 8, 2, 1, "softmax", seed=62)
    args = args_for(d)
    traits = traits_for(1)
    args.workspace = torch.empty(M.fused_moe_workspace_size(traits, args), dtype=torch.uint8, device="cuda:0")
    outs = [torch.empty_like(args.a) for _ in range(2)]

    def step(x, ids, w, slot):
        args.a, args.topk_ids, args.topk_weight, args.o = x, ids, w, outs[slot]
        return M.fused_moe(traits, args, stream=torch.cuda.current_stream())
    n = 5
    batches = [O.f32_to_bf16(O.normal((128, 512), 80 + i, 1)) for i in range(n)]
    x_h = torch.from_numpy(batches[0].view(np.int16).copy()).view(torch.bfloat16).pin_memory()
    ids_h = torch.from_numpy(d["topk_ids"]).pin_memory()
    w_h = torch.from_numpy(d["topk_w"]).pin_memory()
    out_h = torch.empty(128, 512, dtype=torch.bfloat16).pin_memory()
    pipe = api.GraphPipeline(step, x_h, ids_h, w_h, out_h, torch.device("cuda:0"))
    got = []
    for i in range(n):
        if i + 1 < n:
            x_h.copy_(torch.from_numpy(batches[i + 1].view(np.int16).copy()).view(torch.bfloat16))
        pipe.submit()
        pipe.main.synchronize()
        if i > 0:
            got.append(out_h.view(torch.int16).numpy().view(np.uint16).copy())
    pipe.flush()
    got.append(out_h.view(torch.int16).numpy().view(np.uint16).copy())
    for i in range(n):
        di = dict(d, x=batches[i])
        check(di, got[i], run_oracle(di))


@pytest.mark.parametrize("quant", [0, 1])
@pytest.mark.parametrize("T,H,I,E,K", [(128, 512, 512, 8, 2), (16, 256, 256, 4, 2), (700, 256, 768, 3, 1)])
def test_gate_only_variant(quant, T, H, I, E, K):
    """W1 = [E, I, H] without an up projection: y = SiLU(x . W1^T)."""
    d = O.make_inputs(T, H, I, E, K, quant, "softmax", seed=71, gate_only=True)
    tr = traits_for(quant)
    tr.gate_only = 1
    args = args_for(d)
    out = M.fused_moe(tr, args)
    torch.cuda.synchronize()
    assert api.check_status(args.workspace) == 0
    ref = O.fused_moe(d["x"], d["w1"], d["w2"], d["topk_ids"], d["topk_w"], quant, d["w1_scale"], d["w2_scale"],
                      gate_only=True)
    check(d, out_bits(out), ref)
