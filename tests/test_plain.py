"""The plain implementation against the reference's own model code (golden outputs made on the
CPU by tests/golden/make_golden.py), and against itself."""
import json
import os

import pytest
import torch

import plain_llama as pl
from conftest import golden
from golden.make_golden import golden_weights


def _cfg_from(c: dict, tmp_path) -> dict:
    d = dict(c, architectures=["LlamaForCausalLM"])
    with open(os.path.join(tmp_path, "config.json"), "w") as f:
        json.dump(d, f)
    return pl.read_config(str(tmp_path))


@pytest.mark.parametrize("name", ["tiny_a", "tiny_b"])
def test_plain_matches_reference_model(name, tmp_path):
    g = golden(name)
    cfg = _cfg_from(g["config"], tmp_path)
    W = golden_weights(g["config"], g["seed"])
    logits = pl.forward(cfg, W, g["prompt"])
    want = torch.tensor(g["logits"])
    got = logits[g["positions"]]
    # float32 on both sides; only the order of sums differs
    assert (got - want).abs().max().item() < 2e-5 * max(1.0, want.abs().max().item())
    assert g["reference_cut_vs_whole_max_abs"] < 1e-5


def test_prefix_property(tmp_path):
    """Causality: logits of a prefix do not change when tokens are appended."""
    g = golden("tiny_a")
    cfg = _cfg_from(g["config"], tmp_path)
    W = golden_weights(g["config"], g["seed"])
    full = pl.forward(cfg, W, g["prompt"])
    part = pl.forward(cfg, W, g["prompt"][:9])
    assert torch.allclose(full[:9], part, atol=1e-5)


def test_window_limits_keys():
    torch.manual_seed(0)
    q, k, v = torch.randn(12, 4, 16), torch.randn(12, 2, 16), torch.randn(12, 2, 16)
    full = pl.causal_attention(q, k, v, 0.25)
    win = pl.causal_attention(q, k, v, 0.25, window=5)
    assert torch.allclose(full[:5], win[:5], atol=1e-6)          # the first 5 queries see everything
    assert not torch.allclose(full[8:], win[8:], atol=1e-3)
    # the last query with window 5 sees exactly keys 7..11
    alone = pl.causal_attention(q[7:], k[7:], v[7:], 0.25)
    assert torch.allclose(alone[-1], win[-1], atol=1e-6)


def test_rope_is_a_rotation():
    ang = pl.rope_angles(torch.arange(7), 16, 10000.0)
    x = torch.randn(7, 3, 16)
    y = pl.apply_rope(x, ang)
    assert torch.allclose(x.norm(dim=-1), y.norm(dim=-1), atol=1e-5)
    assert torch.allclose(y[0], x[0])                             # position 0: no rotation
    # relative property: <rope(q, m), rope(k, n)> depends on m - n only
    q, k = torch.randn(1, 1, 16), torch.randn(1, 1, 16)
    a = (pl.apply_rope(q, pl.rope_angles(torch.tensor([5]), 16, 1e4)) *
         pl.apply_rope(k, pl.rope_angles(torch.tensor([2]), 16, 1e4))).sum()
    b = (pl.apply_rope(q, pl.rope_angles(torch.tensor([9]), 16, 1e4)) *
         pl.apply_rope(k, pl.rope_angles(torch.tensor([6]), 16, 1e4))).sum()
    assert abs(a - b) < 1e-4


def test_sampling_uniform_and_greedy():
    us = [pl.uniform(3, 7, 2, t) for t in range(2000)]
    assert all(0.0 < u < 1.0 for u in us)
    assert 0.45 < sum(us) / len(us) < 0.55
    assert pl.uniform(3, 7, 2, 5) != pl.uniform(3, 7, 3, 5) != pl.uniform(4, 7, 3, 5)
    lg = torch.tensor([0.1, 2.0, 2.0, -1.0])
    assert pl.sample(lg, 0.0, 0, 0, 0) == 1                       # lowest index wins the tie
    # a sampled token is always one the distribution supports
    lg = torch.tensor([0.0, -1e9, 1.0])
    assert all(pl.sample(lg, 1.0, 5, r, 0) in (0, 2) for r in range(50))


def test_sampling_follows_softmax():
    lg = torch.tensor([1.0, 0.0, -1.0, 0.5])
    t = 0.7
    p = torch.softmax(lg / t, -1)
    n = 4000
    counts = torch.zeros(4)
    for r in range(n):
        counts[pl.sample(lg, t, 1, r, 0)] += 1
    assert (counts / n - p).abs().max() < 0.03
