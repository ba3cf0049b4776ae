"""The plain implementation against the anchors under tests/golden/ (made by the reference's
own CPU oracle, scripts/ref_engine.py in its never-rounding mode), and its own consistency."""
import os

import numpy as np
import pytest
import torch

import plain_llama as plain
from golden.make_golden import GOLDEN, golden_tokens, golden_weights

HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.mark.parametrize("name", ["tiny_a", "tiny_b"])
def test_plain_matches_reference_oracle(name):
    z = np.load(os.path.join(HERE, "golden", name + ".npz"))
    tokens = z["tokens"].tolist()
    assert tokens == golden_tokens(name)
    got = plain.forward(GOLDEN[name]["cfg"], golden_weights(name), tokens)
    ref = torch.from_numpy(z["logits"])
    assert got.shape == ref.shape
    assert float((got - ref).abs().max()) <= 2e-6 * float(ref.abs().max()) + 1e-7


def test_float64_agrees_with_float32():
    name = "tiny_b"
    w32 = golden_weights(name)
    w64 = {k: v.double() for k, v in w32.items()}
    toks = golden_tokens(name)
    a, b = plain.forward(GOLDEN[name]["cfg"], w32, toks), plain.forward(GOLDEN[name]["cfg"], w64, toks)
    assert b.dtype == torch.float64
    assert float((a.double() - b).abs().max()) < 1e-5 * float(b.abs().max())


def test_causality_and_window():
    """A later token does not change earlier logits; a window hides keys that fall out of it."""
    name = "tiny_a"
    cfg, w, toks = GOLDEN[name]["cfg"], golden_weights(name), golden_tokens(name)
    full = plain.forward(cfg, w, toks)
    cut = plain.forward(cfg, w, toks[:9])
    assert torch.allclose(full[:9], cut, atol=1e-6)
    win = plain.forward(cfg, w, toks, window=4)
    assert torch.allclose(win[:4], full[:4], atol=1e-6) and not torch.allclose(win[8:], full[8:], atol=1e-4)


def test_llama3_scaling_bands():
    sc = dict(rope_type="llama3", factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0,
              original_max_position_embeddings=8192)
    base = plain.rope_inv_freq(128, 500000.0)
    scaled = plain.rope_inv_freq(128, 500000.0, sc)
    wavelen = 2 * np.pi / base.double()
    short, long_ = wavelen < 8192 / 4, wavelen > 8192 / 1
    assert torch.equal(scaled[short], base[short])
    assert torch.allclose(scaled[long_], base[long_] / 8)
    mid = ~(short | long_)
    assert bool(mid.any()) and bool(((scaled[mid] < base[mid]) & (scaled[mid] > base[mid] / 8)).all())


def test_greedy_rules_and_sampling_noise():
    assert plain.argmax_lowest(torch.tensor([1.0, 3.0, 3.0])) == 1
    assert plain.argmax_lowest(torch.tensor([1.0, float("nan"), 9.0])) == 1
    assert plain.argmax_lowest(torch.full((4,), float("-inf"))) == 0
    us = [plain.sample_uniform(4, 10, i) for i in range(2000)]
    assert 0 < min(us) and max(us) < 1 and abs(sum(us) / 2000 - 0.5) < 0.03
    assert plain.sample_uniform(4, 10, 3) != plain.sample_uniform(4, 11, 3) != plain.sample_uniform(5, 11, 3)
    # the draws follow softmax(logits / T)
    logits = torch.tensor([2.0, 1.0, 0.0, -1.0])
    counts = torch.zeros(4)
    for pos in range(3000):
        counts[plain.sample_temperature(logits, 0.8, 7, pos)] += 1
    want = torch.softmax(logits / 0.8, 0)
    assert float((counts / 3000 - want).abs().max()) < 0.03
