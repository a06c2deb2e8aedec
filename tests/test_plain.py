"""The plain implementation against closed forms, so that the oracle itself is checked (no GPU)."""
import math

import numpy as np
import torch

import helpers as H
import plain_qwen3 as P


def test_rms_norm_of_a_constant_vector():
    x = torch.full((2, 8), 3.0)
    out = P.rms_norm(x, torch.arange(8.0), 0.0)
    assert torch.allclose(out, torch.arange(8.0).expand(2, 8))
    assert torch.allclose(P.rms_norm(x, torch.ones(8), 16.0), torch.full((2, 8), 3.0 / 5.0))


def test_rotation_is_identity_at_position_zero_and_keeps_norms():
    x = torch.randn(3, 2, 8)
    assert torch.allclose(P.rope(x, [0, 0, 0], 10000.0), x)
    y = P.rope(x, [5, 17, 400], 10000.0)
    assert torch.allclose(y.norm(dim=-1), x.norm(dim=-1), atol=1e-5)
    # the pair (i, i + d/2) turns by pos * theta^(-2i/d)
    e = torch.zeros(1, 1, 8); e[0, 0, 1] = 1.0
    r = P.rope(e, [3], 100.0)
    a = 3 * 100.0 ** (-2 / 8)
    assert torch.allclose(r[0, 0, 1], torch.tensor(math.cos(a)), atol=1e-6)
    assert torch.allclose(r[0, 0, 5], torch.tensor(math.sin(a)), atol=1e-6)


def test_scores_depend_on_relative_positions_only():
    q, k = torch.randn(1, 1, 16), torch.randn(1, 1, 16)
    a = (P.rope(q, [9], 1e4) * P.rope(k, [4], 1e4)).sum()
    b = (P.rope(q, [109], 1e4) * P.rope(k, [104], 1e4)).sum()
    assert torch.allclose(a, b, atol=1e-4)


def test_attention_is_causal_and_groups_heads_in_blocks():
    P_, nq, nkv, d = 6, 4, 2, 8
    q, k, v = torch.randn(P_, nq, d), torch.randn(P_, nkv, d), torch.randn(P_, nkv, d)
    out = P.causal_attention(q, k, v)
    assert torch.allclose(out[0, 0], v[0, 0]) and torch.allclose(out[0, 3], v[0, 1])   # one key: returns v
    k2, v2 = k.clone(), v.clone()
    k2[4:], v2[4:] = 9.0, -9.0                                                       # the future does not matter
    assert torch.allclose(P.causal_attention(q, k2, v2)[:4], out[:4])
    same = P.causal_attention(torch.zeros(P_, nq, d), k, v)                         # equal scores average v
    assert torch.allclose(same[3, 1], v[:4, 0].mean(0), atol=1e-6)
    win = P.causal_attention(q, k, v, window=2)
    assert torch.allclose(win[5], P.causal_attention(q[4:], k[4:], v[4:])[1], atol=1e-6)


def test_forward_prefix_property_and_tied_head():
    cfg, w = H.plain_model("A")
    toks = H.tokens_for("A", 12, 0)
    full = P.forward(cfg, w, toks)
    assert full.shape == (12, 256)
    assert torch.allclose(P.forward(cfg, w, toks[:7]), full[:7], atol=1e-6)
    cfg_b, w_b = H.plain_model("B")
    assert "lm_head.weight" in w_b and "lm_head.weight" not in w
    assert P.forward(cfg_b, w_b, H.tokens_for("B", 5, 0)).shape == (5, 333)


def test_sampling_functions():
    logits = [0.5, 2.0, 2.0, -1.0, float("nan")]
    assert P.argmax([1.0, 3.0, 3.0]) == 1
    assert P.top_k_mask([1.0, 3.0, 2.0, 3.0], 2) == [-math.inf, 3.0, -math.inf, 3.0]
    assert P.apply_repeat_penalty([2.0, -2.0, 1.0], [0, 1, 1], 2.0) == [1.0, -4.0, 1.0]
    assert P.apply_presence_penalty([2.0, -2.0, 1.0], [0, 0], 0.5) == [1.5, -2.0, 1.0]
    assert P.apply_logit_bias([0.0, 0.0], {1: 3.0, 9: 1.0}) == [0.0, 3.0]
    p = P.temperature_probs(logits, 1.0)
    assert p[4] == 0 and abs(p.sum() - 1) < 1e-12 and p[1] == p[2]
    assert P.temperature_sample(logits, 1.0, 0.0) == 0 and P.temperature_sample(logits, 1.0, 0.999999) == 3
    assert P.temperature_sample(logits, 0.0, 0.3) == 1
    keep = P.top_p_keep([0.0, 3.0, 1.0, 2.0], 0.8)
    assert keep == [1, 3]


def test_plain_implementation_reproduces_its_committed_numbers():
    """tests/golden/plain_tiny.json (written by tests/golden/make_plain_golden.py) pins the oracle and
    the seeded weights: an edit to either shows here instead of moving every comparison silently."""
    import json
    from pathlib import Path
    golden = json.loads((Path(__file__).resolve().parent / "golden" / "plain_tiny.json").read_text())
    for which, want in golden.items():
        cfg, w = H.plain_model(which)
        assert H.tokens_for(which, len(want["tokens"]), 7) == want["tokens"]
        logits = P.forward(cfg, w, want["tokens"], dtype=torch.float64)
        scale = float(logits.abs().max())
        assert np.allclose(logits[0, :8].numpy(), want["first"], atol=1e-9 * scale, rtol=1e-7)
        assert np.allclose(logits[-1, :8].numpy(), want["last"], atol=1e-9 * scale, rtol=1e-7)
        assert math.isclose(float((logits * logits).sum()), want["sum_squares"], rel_tol=1e-9)
        assert abs(float(logits.sum()) - want["sum"]) <= 1e-9 * scale * logits.numel()
