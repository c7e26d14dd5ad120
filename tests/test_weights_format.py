"""CPU tests of the on-disk expert-weight format and of the quantisation helpers against
the oracle's definition."""
import numpy as np
import torch

from oracle import oracle as O
from therock_b200 import weights as W


def test_quantize_experts_matches_oracle_definition():
    w = torch.from_numpy(O.normal((3, 256, 384), 4, 2, 0.02))
    q, s = W.quantize_experts(w, "token_channel")
    rq, rs = O.quant_rows_e4m3(w.numpy().reshape(3 * 256, 384))
    assert (q.numpy().reshape(3 * 256, 384) == rq).all()
    assert (s.numpy().reshape(-1) == rs.reshape(-1)).all()
    qb, sb = W.quantize_experts(w, "block128")
    for e in range(3):
        rq, rs = O.quant_blocks_e4m3(w[e].numpy())
        assert (qb[e].numpy() == rq).all() and (sb[e].numpy() == rs).all()
    b, none = W.quantize_experts(w, "none")
    assert none is None and (b.view(torch.int16).numpy().view(np.uint16) == O.f32_to_bf16(w.numpy())).all()


def test_save_load_roundtrip_and_expert_shard(tmp_path):
    w1 = torch.from_numpy(O.normal((4, 512, 256), 5, 2, 0.02))
    w2 = torch.from_numpy(O.normal((4, 256, 256), 5, 3, 0.02))
    for mode in ("none", "token_channel", "block128"):
        q1, s1 = W.quantize_experts(w1, mode)
        q2, s2 = W.quantize_experts(w2, mode)
        path = str(tmp_path / f"layer_{mode}.fmoe")
        W.save_expert_weights(path, q1, q2, mode, s1, s2)
        full = W.load_expert_weights(path)
        assert full["quant"] == mode
        assert torch.equal(full["w1"].view(torch.uint8), q1.view(torch.uint8))
        assert torch.equal(full["w2"].view(torch.uint8), q2.view(torch.uint8))
        if mode != "none":
            assert torch.equal(full["w1_scale"], s1) and torch.equal(full["w2_scale"], s2)
        shard = W.load_expert_weights(path, experts=range(2, 4))
        assert torch.equal(shard["w1"].view(torch.uint8), q1[2:4].view(torch.uint8))
        assert shard["w2"].shape[0] == 2


def test_tile_untile_roundtrip_and_tile_contiguity():
    w = torch.arange(2 * 256 * 384, dtype=torch.int32).view(2, 256, 384).to(torch.bfloat16)
    t = W.tile_weights(w)
    assert t.shape == w.shape and torch.equal(W.untile_weights(t), w)
    # tile (expert 1, row block 1, K block 2) is one contiguous run of 128 x 64 elements
    flat = t.reshape(-1)
    kb = 384 // 64
    start = ((1 * 2 + 1) * kb + 2) * 128 * 64
    assert torch.equal(flat[start:start + 128 * 64].view(128, 64), w[1, 128:256, 128:192])
    q = torch.randint(0, 255, (3, 128, 256), dtype=torch.uint8)
    assert torch.equal(W.untile_weights(W.tile_weights(q)), q)
