"""Checks of the plain implementation itself (CPU)."""
import math

import pytest
import torch

from conftest import TINY_A, TINY_B, TINY_C, random_tokens
from plain_minicpm import (plain_attention, plain_forward, plain_greedy, plain_rmsnorm, plain_rope,
                           plain_sample, plain_scales, plain_swiglu_ffn)


def test_rotate_half_on_checkpoint_rows_equals_adjacent_pairs_on_the_reference_permutation():
    """scripts/jiuge.py:217-227 permutes the rows of W_q / W_k inside each head as
    reshape(h, 2, dh/2, d).transpose(1, 2) and the rotary operator turns pairs (2j, 2j+1).
    Scores q.k are the same as with rotate-half on the unpermuted rows."""
    torch.manual_seed(0)
    T, H, dh, d, theta = 9, 3, 16, 24, 10000.0
    h = torch.randn(T, d, dtype=torch.float64)
    wq, wk = torch.randn(H * dh, d, dtype=torch.float64), torch.randn(H * dh, d, dtype=torch.float64)
    pos = torch.arange(T) + 5
    q = plain_rope((h @ wq.T).view(T, H, dh), pos, theta)
    k = plain_rope((h @ wk.T).view(T, H, dh), pos, theta)

    def permute(w):
        return w.reshape(H, 2, dh // 2, d).transpose(1, 2).reshape(H * dh, d)

    def adjacent(x):
        j = torch.arange(dh // 2, dtype=torch.float64)
        ang = pos.to(torch.float64)[:, None] / theta ** (j / (dh // 2))
        c, s = ang.cos()[:, None, :], ang.sin()[:, None, :]
        x0, x1 = x[..., 0::2], x[..., 1::2]
        out = torch.empty_like(x)
        out[..., 0::2] = x0 * c - x1 * s
        out[..., 1::2] = x0 * s + x1 * c
        return out

    q2 = adjacent((h @ permute(wq).T).view(T, H, dh))
    k2 = adjacent((h @ permute(wk).T).view(T, H, dh))
    s1 = torch.einsum("ihd,jhd->hij", q, k)
    s2 = torch.einsum("ihd,jhd->hij", q2, k2)
    assert torch.allclose(s1, s2, atol=1e-12)


def test_rope_depends_on_relative_position_only():
    torch.manual_seed(1)
    q, k = torch.randn(1, 1, 32, dtype=torch.float64), torch.randn(1, 1, 32, dtype=torch.float64)
    def score(pq, pk):
        return float((plain_rope(q, torch.tensor([pq]), 1e4) * plain_rope(k, torch.tensor([pk]), 1e4)).sum())
    assert math.isclose(score(7, 3), score(107, 103), rel_tol=1e-9)
    assert not math.isclose(score(7, 3), score(7, 4), rel_tol=1e-3)


def test_rmsnorm_and_swiglu_formulas():
    x = torch.tensor([[3.0, 4.0]], dtype=torch.float64)
    w = torch.tensor([2.0, 0.5], dtype=torch.float64)
    y = plain_rmsnorm(x, w, 0.0)
    assert torch.allclose(y, torch.tensor([[3 / math.sqrt(12.5) * 2, 4 / math.sqrt(12.5) * 0.5]], dtype=torch.float64))
    h = torch.tensor([[1.0]], dtype=torch.float64)
    out = plain_swiglu_ffn(h, torch.tensor([[2.0]], dtype=torch.float64), torch.tensor([[3.0]], dtype=torch.float64),
                           torch.tensor([[5.0]], dtype=torch.float64))
    assert math.isclose(float(out), 2 / (1 + math.exp(-2)) * 3 * 5)


def test_attention_is_causal_grouped_and_windowed():
    torch.manual_seed(2)
    T, nh, nkvh, dh = 12, 6, 2, 8
    q = torch.randn(T, nh, dh, dtype=torch.float64)
    k = torch.randn(T, nkvh, dh, dtype=torch.float64)
    v = torch.randn(T, nkvh, dh, dtype=torch.float64)
    out = plain_attention(q, k, v, dh ** -0.5)
    # row 0 sees only itself
    assert torch.allclose(out[0], v[0].repeat_interleave(nh // nkvh, dim=0))
    # later keys do not matter
    k2, v2 = k.clone(), v.clone()
    k2[8:] += 1.0; v2[8:] -= 2.0
    assert torch.allclose(plain_attention(q, k2, v2, dh ** -0.5)[:8], out[:8])
    # grouped heads = repeated heads
    rep = plain_attention(q, k.repeat_interleave(3, 1), v.repeat_interleave(3, 1), dh ** -0.5)
    assert torch.allclose(rep, out)
    # a window at least as long as the sequence changes nothing; a short one does
    assert torch.allclose(plain_attention(q, k, v, dh ** -0.5, window=T), out)
    win = plain_attention(q, k, v, dh ** -0.5, window=3)
    assert torch.allclose(win[:3], out[:3]) and not torch.allclose(win[5], out[5])
    one = plain_attention(q, k, v, dh ** -0.5, window=1)
    assert torch.allclose(one, v.repeat_interleave(3, 1))


@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_logits_are_causal_and_stable_across_precisions(tiny_models, name):
    _, cfg, w = tiny_models[name]
    toks = random_tokens(3, 24, cfg["vocab_size"])
    full = plain_forward(cfg, w, toks)
    assert full.shape == (24, cfg["vocab_size"]) and torch.isfinite(full).all()
    part = plain_forward(cfg, w, toks[:10])
    assert torch.allclose(full[:10], part, atol=1e-10)
    f32 = plain_forward(cfg, w, toks, dtype=torch.float32)
    assert (f32.double() - full).abs().max() <= 2e-4 * full.abs().max()


def test_scales_change_the_function(tiny_models):
    _, cfg, w = tiny_models["A"]
    toks = random_tokens(4, 8, cfg["vocab_size"])
    a = plain_forward(cfg, w, toks)
    b = plain_forward(dict(cfg, model_type="llama"), w, toks)
    assert plain_scales(dict(cfg, model_type="llama")) == (1.0, 1.0, 1.0)
    assert not torch.allclose(a, b, atol=1e-3)
    c = plain_forward(dict(cfg, logit_scale=8.0), w, toks)
    assert torch.allclose(c, a * 2.0, atol=1e-10)       # tiny-A's own logit scale is 4


def test_tied_and_untied_output(tiny_models):
    _, cfg, w = tiny_models["A"]
    assert "lm_head.weight" not in w
    w2 = dict(w, **{"lm_head.weight": w["model.embed_tokens.weight"].clone()})
    toks = random_tokens(5, 6, cfg["vocab_size"])
    assert torch.equal(plain_forward(cfg, w, toks), plain_forward(cfg, w2, toks))
    assert "lm_head.weight" in tiny_models["B"][2]


def test_run_order_a_layer_twice_and_a_shared_cache(tiny_models):
    _, cfg, w = tiny_models["A"]
    toks = random_tokens(6, 10, cfg["vocab_size"])
    base = plain_forward(cfg, w, toks)
    same = plain_forward(cfg, w, toks, order=[(0, 0, True), (1, 1, True)])
    assert torch.equal(base, same)
    twice = plain_forward(cfg, w, toks, order=[(0, 0, True), (1, 1, True), (0, 2, True)])
    shared = plain_forward(cfg, w, toks, order=[(0, 0, True), (1, 0, False)])
    assert not torch.allclose(twice, base, atol=1e-4) and not torch.allclose(shared, base, atol=1e-4)


def test_greedy_continues_itself(tiny_models):
    _, cfg, w = tiny_models["B"]
    prompt = random_tokens(7, 5, cfg["vocab_size"])
    out = plain_greedy(cfg, w, prompt, 4)
    assert plain_greedy(cfg, w, prompt + out[:2], 2) == out[2:]


def test_sampling_rule():
    logits = torch.tensor([1.0, 3.0, 2.0, 3.0, -1.0])
    assert plain_sample(logits, 0.0, 0, 1.0, 0.9) == 1           # greedy: first of the equal maxima
    assert plain_sample(logits, 1.0, 1, 1.0, 0.9) == 1           # topk 1 is greedy
    w = torch.exp(logits.double() - 3.0)
    cdf = torch.cumsum(w, 0) / w.sum()
    for u in (0.0, 0.05, 0.3, 0.6, 0.95, 0.999):
        want = int((cdf > u).nonzero()[0])
        assert plain_sample(logits, 1.0, 0, 1.0, u) == want
    # topk 2: only the two 3.0 entries; vocabulary order decides
    assert plain_sample(logits, 1.0, 2, 1.0, 0.1) == 1 and plain_sample(logits, 1.0, 2, 1.0, 0.9) == 3
    # topk 3 reaches down to the 2.0
    assert plain_sample(logits, 1.0, 3, 1.0, 0.5) == 2
    # topp: the two 3.0 carry 2/(2+e^-1+e^-2+e^-4) = 0.79 of the mass
    assert plain_sample(logits, 1.0, 0, 0.7, 0.99) == 3
    assert plain_sample(logits, 1.0, 0, 0.9, 0.55) == 2
    # a low temperature sharpens
    assert plain_sample(logits, 0.05, 0, 1.0, 0.49) == 1 and plain_sample(logits, 0.05, 0, 1.0, 0.51) == 3
