"""The plain implementation itself, against closed forms and its own invariants (no GPU)."""
import math

import numpy as np
import torch

import plain_qwen3 as plain
from helpers import TINY, make_model_dir


def test_rms_norm_closed_form():
    x = torch.tensor([[3.0, 4.0]], dtype=torch.float64)
    w = torch.tensor([2.0, 0.5], dtype=torch.float64)
    y = plain.rms_norm(x, w, 0.0)
    r = math.sqrt((9 + 16) / 2)
    assert torch.allclose(y, torch.tensor([[3 / r * 2, 4 / r * 0.5]], dtype=torch.float64))
    assert plain.rms_norm(x, w, 1e-2)[0, 0] < y[0, 0]


def test_rope_is_a_rotation_by_position_times_frequency():
    d, theta = 8, 100.0
    pos = torch.tensor([0, 3, 7])
    cos, sin = plain.rope_tables(pos, d, theta)
    assert cos.shape == (3, 4) and torch.allclose(cos[0], torch.ones(4, dtype=torch.float64))
    assert math.isclose(float(sin[1, 1]), math.sin(3 * theta ** (-2 / 8)))
    x = torch.randn(3, 2, d, dtype=torch.float64)
    y = plain.apply_rope(x, cos, sin)
    assert torch.allclose(y.norm(dim=-1), x.norm(dim=-1))             # rotations keep lengths
    assert torch.allclose(y[0], x[0])                                 # position 0: identity
    # pair (i, i + d/2) is rotated together
    i = 1
    a = 3 * theta ** (-2 * i / d)
    assert math.isclose(float(y[1, 0, i]), float(x[1, 0, i] * math.cos(a) - x[1, 0, i + 4] * math.sin(a)))
    assert math.isclose(float(y[1, 0, i + 4]), float(x[1, 0, i + 4] * math.cos(a) + x[1, 0, i] * math.sin(a)))
    # scores depend on the distance only
    q = torch.randn(1, 1, d, dtype=torch.float64).expand(3, 1, d)
    k = torch.randn(1, 1, d, dtype=torch.float64).expand(3, 1, d)
    c2, s2 = plain.rope_tables(pos + 11, d, theta)
    s_a = (plain.apply_rope(q, cos, sin)[2, 0] * plain.apply_rope(k, cos, sin)[1, 0]).sum()
    s_b = (plain.apply_rope(q, c2, s2)[2, 0] * plain.apply_rope(k, c2, s2)[1, 0]).sum()
    assert math.isclose(float(s_a), float(s_b), rel_tol=1e-9)


def test_attention_is_causal_grouped_and_windowed():
    T, nh, nkv, d = 9, 4, 2, 6
    q, k, v = (torch.randn(T, n, d, dtype=torch.float64) for n in (nh, nkv, nkv))
    out = plain.causal_attention(q, k, v, 0.3)
    assert torch.allclose(out[0, :, :], v[0, [0, 0, 1, 1], :])        # first token sees itself only; head h -> kv h // 2
    k2, v2 = k.clone(), v.clone()
    k2[5:], v2[5:] = 7.0, -3.0
    assert torch.allclose(plain.causal_attention(q, k2, v2, 0.3)[:5], out[:5])   # the future does not matter
    # one key made to stand out takes all the weight
    k3 = k.clone()
    k3[2, 0] = q[8, 0] * 50
    o3 = plain.causal_attention(q, k3, v, 1.0)
    assert torch.allclose(o3[8, 0], v[2, 0], atol=1e-6)
    # a window of 3 sees keys i-2 .. i: the standing-out key at 2 is gone for query 8 but there for query 4
    k3[2, 0] = q[4, 0] * 50
    ow = plain.causal_attention(q, k3, v, 1.0, window=3)
    assert torch.allclose(ow[4, 0], v[2, 0], atol=1e-6)
    full = plain.causal_attention(q[6:9], k[6:9], v[6:9], 1.0)
    assert torch.allclose(ow[8], full[2], atol=1e-12)                 # query 8 sees exactly keys 6, 7, 8


def test_forward_of_a_prefix_equals_the_prefix_of_the_forward(tmp_path):
    d = make_model_dir(str(tmp_path), "C")
    cfg, w = plain.read_model(d)
    toks = np.random.default_rng(0).integers(0, cfg["vocab_size"], 60).tolist()
    full = plain.forward(cfg, w, toks)
    part = plain.forward(cfg, w, toks[:41])
    assert full.shape == (60, 301) and torch.allclose(full[:41], part, atol=1e-12)
    # the window matters: without it the late logits differ
    cfg2 = dict(cfg)
    del cfg2["layer_types"]
    assert (plain.forward(cfg2, w, toks)[-1] - full[-1]).abs().max() > 1e-4
    assert torch.allclose(plain.forward(cfg2, w, toks)[:37], full[:37], atol=1e-12)


def test_tied_and_untied_heads(tmp_path):
    da, db = make_model_dir(str(tmp_path), "A"), make_model_dir(str(tmp_path), "B")
    ca, wa = plain.read_model(da)
    cb, wb = plain.read_model(db)
    assert "lm_head.weight" not in wa and "lm_head.weight" in wb
    x = torch.randn(2, 64, dtype=torch.float64)
    z = plain.rms_norm(x, wa["model.norm.weight"], 1e-6)
    assert torch.allclose(plain.lm_head(x, wa, ca), z @ wa["model.embed_tokens.weight"].T)


def test_sampler_kept_set_matches_sorted_prefix_rules():
    logits = np.log(np.array([0.5, 0.2, 0.15, 0.1, 0.05]))
    kept, p = plain.sample_kept_set(logits, 1.0, 0, 1.0, 0.0)
    assert list(kept) == [0, 1, 2, 3, 4] and np.allclose(p, [0.5, 0.2, 0.15, 0.1, 0.05])
    kept, p = plain.sample_kept_set(logits, 1.0, 3, 1.0, 0.0)
    assert list(kept) == [0, 1, 2] and np.allclose(p, np.array([0.5, 0.2, 0.15]) / 0.85)
    kept, _ = plain.sample_kept_set(logits, 1.0, 0, 0.7, 0.0)           # 0.5 + 0.2 reaches 0.7
    assert list(kept) == [0, 1]
    kept, _ = plain.sample_kept_set(logits, 1.0, 0, 0.71, 0.0)
    assert list(kept) == [0, 1, 2]
    kept, _ = plain.sample_kept_set(logits, 1.0, 0, 1.0, 0.25)          # p >= 0.125
    assert list(kept) == [0, 1, 2]
    kept, _ = plain.sample_kept_set(logits, 0.5, 0, 1.0, 0.25)          # temperature sharpens: p^2 >= 0.25 * 0.25
    assert list(kept) == [0]
