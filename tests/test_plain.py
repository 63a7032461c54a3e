"""The plain implementation checked against itself and against independent restatements (no GPU)."""
import math

import pytest
import torch

import plain_model
from tiny import TINY, random_tokens


def test_float32_and_float64_agree(model_dirs):
    for name in ("A", "B"):
        toks = random_tokens(40, TINY[name]["vocab_size"], 3)
        a = plain_model.forward(model_dirs[name], toks)
        b = plain_model.forward(model_dirs[name], toks, compute=torch.float64)
        assert float((a - b.float()).abs().max()) < 5e-6


def test_causal_a_prefix_does_not_see_what_follows(model_dirs):
    toks = random_tokens(30, 256, 4)
    whole = plain_model.forward(model_dirs["A"], toks, compute=torch.float64)
    prefix = plain_model.forward(model_dirs["A"], toks[:11], compute=torch.float64)
    assert float((whole[:11] - prefix).abs().max()) < 1e-12


def test_window_drops_old_keys(model_dirs):
    """Model B's later layers see 40 positions: a change at position 0 cannot reach position 90
    through them, but it does through layer 0, so only a windowless variant differs more."""
    toks = random_tokens(96, 384, 5)
    other = [(toks[0] + 1) % 384] + toks[1:]
    a = plain_model.forward(model_dirs["B"], toks, compute=torch.float64)
    b = plain_model.forward(model_dirs["B"], other, compute=torch.float64)
    assert float((a[95] - b[95]).abs().max()) > 0            # layer 0 sees every key
    # attention alone: with a window of 40 the query at 90 ignores key 0
    q = torch.randn(96, 3, 32, dtype=torch.float64); k = torch.randn(96, 1, 32, dtype=torch.float64); v = torch.randn(96, 1, 32, dtype=torch.float64)
    k2, v2 = k.clone(), v.clone(); k2[0] += 5; v2[0] += 5
    w = plain_model.attend(q, k, v, 3, 1, 40); w2 = plain_model.attend(q, k2, v2, 3, 1, 40)
    assert torch.equal(w[40:], w2[40:]) and not torch.equal(w[39], w2[39])
    f = plain_model.attend(q, k, v, 3, 1, None); f2 = plain_model.attend(q, k2, v2, 3, 1, None)
    assert not torch.equal(f[90], f2[90])


def test_attend_matches_a_restatement_with_softmax():
    torch.manual_seed(0)
    n, heads, kv_heads, hd = 9, 4, 2, 16
    q, k, v = torch.randn(n, heads, hd), torch.randn(n, kv_heads, hd), torch.randn(n, kv_heads, hd)
    got = plain_model.attend(q, k, v, heads, kv_heads, None)
    kk, vv = k.repeat_interleave(2, dim=1), v.repeat_interleave(2, dim=1)
    scores = torch.einsum("qhd,khd->hqk", q, kk) / math.sqrt(hd)
    scores = scores.masked_fill(torch.triu(torch.ones(n, n, dtype=torch.bool), 1), float("-inf"))
    want = torch.einsum("hqk,khd->qhd", torch.softmax(scores, dim=-1), vv)
    assert float((got - want).abs().max()) < 1e-5


def test_rope_is_a_rotation_by_position_times_frequency():
    cos, sin = plain_model.rope_tables(50, 8, 10000.0)
    x = torch.zeros(50, 1, 8); x[:, 0, 1] = 1.0          # unit vector on element 1, whose pair is element 5
    y = plain_model.rope(x, cos, sin)
    for pos in (0, 1, 17, 49):
        angle = pos * 10000.0 ** (-2 / 8)
        assert abs(float(y[pos, 0, 1]) - math.cos(angle)) < 1e-6 and abs(float(y[pos, 0, 5]) - math.sin(angle)) < 1e-6
    assert float((y.norm(dim=-1) - 1).abs().max()) < 1e-6


def test_rmsnorm_and_swiglu_formulas():
    x, w = torch.tensor([[3.0, 4.0]]), torch.tensor([2.0, 0.5])
    inv = 1 / math.sqrt(12.5 + 1e-6)
    assert torch.allclose(plain_model.rmsnorm(x, w, 1e-6), torch.tensor([[3 * inv * 2, 4 * inv * 0.5]]))
    g, u = torch.tensor([0.0, 2.0]), torch.tensor([3.0, 3.0])
    assert torch.allclose(plain_model.swiglu(g, u), torch.tensor([0.0, 3 * 2 / (1 + math.exp(-2))]))


def test_argmax_ties_go_to_the_lowest_id_and_bans_hold():
    assert plain_model.argmax([1.0, 3.0, 3.0, 2.0]) == 1
    assert plain_model.argmax([1.0, 3.0, 3.0, 2.0], banned=[0, 1, 0, 0]) == 2


def test_sampler_rules():
    torch.manual_seed(1)
    logits = torch.randn(60).tolist()
    # top-k 1 at any temperature is greedy (tests/runtime.test.ts:133-152 of the reference)
    assert plain_model.sample(logits, 0.9, 1, 1.0, 1)[0] == plain_model.argmax(logits)
    # a fixed seed repeats; the state advances once per draw
    a = plain_model.sample(logits, 0.8, 40, 0.95, 1)
    assert a == plain_model.sample(logits, 0.8, 40, 0.95, 1) and a[1] == plain_model.xorshift32(1)
    draws = set()
    state = 12345
    for _ in range(200):
        tok, state = plain_model.sample(logits, 1.5, 0, 1.0, state)
        draws.add(tok)
    assert len(draws) > 10
    # top-p keeps the shortest prefix: with a tiny top_p only the best token is left
    assert all(plain_model.sample(logits, 1.0, 0, 1e-6, s)[0] == plain_model.argmax(logits) for s in (1, 2, 3))
    # banned ids never come
    banned = [0] * 60; banned[plain_model.argmax(logits)] = 1
    assert all(plain_model.sample(logits, 0.5, 3, 0.9, s, banned)[0] != plain_model.argmax(logits) for s in range(1, 30))
