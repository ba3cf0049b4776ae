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


LLAMA3_PINNED = {
    # (head_dim, theta, factor, low, high, original): {index: (inv_freq, band)}. The values were worked out once from
    # the rule itself in 50-digit decimal arithmetic, outside every implementation compared here: unscaled
    # frequency f = theta^(-2i/D), wavelength 2 pi / f; kept below original/high, divided by factor above
    # original/low, between them f * ((1 - s) / factor + s) with s = (original / wavelength - low) / (high - low).
    (64, 500000.0, 32.0, 1.0, 4.0, 8192): {0: (1.0, "keep"), 1: (0.6636012376960885, "keep"), 15: (0.0012905479282092638, "mid"),
                                           17: (9.708287802627673e-05, "mid"), 18: (1.9461638184831125e-05, "div"),
                                           31: (9.41830672543491e-08, "div")},
    (128, 500000.0, 8.0, 1.0, 4.0, 8192): {0: (1.0, "keep"), 1: (0.8146172338565447, "keep"), 29: (0.0021665707635033587, "mid"),
                                           34: (0.0001785078127679964, "mid"), 35: (9.556212353964683e-05, "div"),
                                           63: (3.068925988914511e-07, "div")},
    (32, 500000.0, 32.0, 1.0, 4.0, 64): {0: (1.0, "keep"), 1: (0.44036660267178046, "keep"), 2: (0.06713303751104989, "mid"),
                                         3: (0.0026686593839301753, "div"), 15: (1.4192720251899592e-07, "div")},
}


def test_llama3_scaling_values_are_pinned():
    """The Llama-3 frequency rule at the 1B's, the 8B's and tiny B's parameters: the product's table builder, the
    plain implementation and the reference arm's writer (three separately written statements of the rule: vectorised
    float64, the same in the tests, scalar Python floats) against values worked out by hand in decimal arithmetic,
    at the first and last index of every band. The reference takes these numbers as data from its exporter
    (scripts/export.py:104-108), so its golden outputs cover their use and this test covers the rule."""
    import os
    import sys

    from hipinfer_b200.parts.rotary import rope_inv_freq

    sys.path.insert(0, os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "baseline"))
    import reference_arm

    for (D, theta, factor, low, high, orig), pins in LLAMA3_PINNED.items():
        sc = dict(rope_type="llama3", factor=factor, low_freq_factor=low, high_freq_factor=high,
                  original_max_position_embeddings=orig)
        ours, plain_v = rope_inv_freq(D, theta, sc), plain.rope_inv_freq(D, theta, sc)
        arm = torch.tensor(reference_arm.llama3_inv_freq(D, theta, sc), dtype=torch.float64)
        assert ours.dtype == torch.float32 and ours.shape == (D // 2,)
        assert torch.equal(ours, plain_v)
        assert float(((arm - ours.double()).abs() / arm).max()) < 1e-7       # float32 rounding of the stored table
        for i, (want, _) in pins.items():
            assert abs(float(ours[i]) - want) <= 6e-8 * want, (D, i, float(ours[i]), want)
            assert abs(float(arm[i]) - want) <= 1e-12 * want, (D, i, float(arm[i]), want)
        # the bands are where the pins say: the count of kept, blended and divided frequencies
        base = plain.rope_inv_freq(D, theta).double()
        ratio = ours.double() / base
        kept, divided = int((ratio > 1 - 1e-6).sum()), int((ratio < 1 / factor + 1e-6).sum())
        first_mid = min(i for i, (_, b) in pins.items() if b == "mid")
        first_div = min(i for i, (_, b) in pins.items() if b == "div")
        assert (kept, divided) == (first_mid, D // 2 - first_div)


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
