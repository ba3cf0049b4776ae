"""Plain, slow implementation of the dense Llama decoder for the tests.

Whole sequences, no cache, one function for each part, CPU only. It shares no code with the
`hipinfer_b200` package: it reads `config.json` and `model.safetensors` with the standard
`json` module and the `safetensors` library, and works on plain torch tensors.

Every function is written from the formulas of Sky1219/hipinfer and cites the place
(`file:line` inside that project) it was read from. The reference rounds to fp16 after most
operations so that it matches a half-precision framework bit for bit (src/kernels.cuh:1-3); its
own oracle has a mode that never rounds (scripts/ref_engine.py:9-10, 137-139). This file is that
never-rounding mode: same operations, same order, computed in `dtype` (float32 by default,
float64 when a test wants a tighter yardstick).

Anchor: `tests/golden/` holds logits that the reference's `scripts/ref_engine.py` (mode "fp32")
produced on tiny random models, with the script that made them; `tests/test_plain.py` compares
this file with them. The Llama-3 frequency scaling itself rests on the formula only, since the
reference takes `inv_freq` as data copied from another framework (scripts/export.py:104-108).
"""
from __future__ import annotations

import json
import math
import os

import torch


# --------------------------------------------------------------------------------------
# model folder
# --------------------------------------------------------------------------------------
def read_model(folder, dtype=torch.float32):
    """(config dict, {tensor name: tensor in `dtype`}) of a folder with config.json and
    model.safetensors. Tensor names are the ones scripts/export.py:221-287 consumes."""
    from safetensors import safe_open

    with open(os.path.join(folder, "config.json")) as f:
        cfg = json.load(f)
    weights = {}
    with safe_open(os.path.join(folder, "model.safetensors"), framework="pt", device="cpu") as f:
        for name in f.keys():
            weights[name] = f.get_tensor(name).to(dtype)
    return cfg, weights


def head_dim_of(cfg):
    """head_dim, or hidden/heads when the key is absent (scripts/export.py:203)."""
    hd = cfg.get("head_dim")
    return int(hd) if hd else cfg["hidden_size"] // cfg["num_attention_heads"]


def kv_heads_of(cfg):
    """num_key_value_heads, or the number of query heads when absent (scripts/layer_diff.py:51)."""
    kv = cfg.get("num_key_value_heads")
    return int(kv) if kv else cfg["num_attention_heads"]


# --------------------------------------------------------------------------------------
# parts
# --------------------------------------------------------------------------------------
def embed(tokens, table):
    """x[i, :] = E[tok[i], :], a row gather without scaling (src/kernels.cuh:1877-1881)."""
    return table[torch.as_tensor(tokens, dtype=torch.long)]


def rmsnorm(x, w, eps):
    """y = w * (x * rsqrt(mean(x^2) + eps)), plain weight, not 1 + w
    (src/kernels.cuh:108-125; scripts/ref_engine.py:145-147)."""
    r = torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps)
    return w * (x * r)


def rope_inv_freq(head_dim, theta, scaling=None):
    """inv_freq[i] = theta^(-2i/D) (scripts/export.py:109-111; tests/test_kernels.py:224-227),
    then, for rope_type "llama3", the per-frequency rescaling by wavelength: short waves kept,
    long waves divided by `factor`, the band between interpolated. The reference copies the
    scaled values from another framework's rotary module (scripts/export.py:104-108), so this
    half of the function rests on the published formula alone. Computed in float64, returned
    as float32, as the reference stores it (src/api.cu:1430-1441 reads an fp32 array)."""
    i = torch.arange(0, head_dim, 2, dtype=torch.float64)
    inv = 1.0 / (float(theta) ** (i / head_dim))
    if scaling:
        kind = scaling.get("rope_type", scaling.get("type"))
        if kind == "llama3":
            factor = float(scaling["factor"])
            low = float(scaling["low_freq_factor"])
            high = float(scaling["high_freq_factor"])
            orig = float(scaling["original_max_position_embeddings"])
            wavelen = 2.0 * math.pi / inv
            smooth = (orig / wavelen - low) / (high - low)
            mid = (1.0 - smooth) * inv / factor + smooth * inv
            inv = torch.where(wavelen < orig / high, inv, torch.where(wavelen > orig / low, inv / factor, mid))
        elif kind not in (None, "default"):
            raise ValueError(f"plain implementation: rope_type {kind!r} is not part of this architecture")
    return inv.to(torch.float32)


def rope_cos_sin(positions, inv_freq, dtype=torch.float32):
    """cos/sin [T, D/2]: the angle float(p) * inv_freq[i] is a float32 product, cos and sin are
    evaluated in double (src/api.cu:1430-1441; scripts/ref_engine.py:152-157). attention_scaling
    is 1 for this architecture."""
    a = torch.as_tensor(positions).to(torch.float32)[:, None] * inv_freq.to(torch.float32)[None, :]
    return torch.cos(a.double()).to(dtype), torch.sin(a.double()).to(dtype)


def apply_rope(x, cos, sin):
    """Half-split pairs (d, d + D/2) over the whole head: y1 = x1 cos - x2 sin,
    y2 = x2 cos + x1 sin (src/kernels.cuh:127-136; scripts/ref_engine.py:159-166).
    x is [T, heads, D]."""
    h = x.shape[-1] // 2
    x1, x2 = x[..., :h], x[..., h:]
    c, s = cos[:, None, :], sin[:, None, :]
    return torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], -1)


def attention_scores_softmax_values(q, k, v, q_pos, k_pos, window=None):
    """Causal softmax attention on absolute positions: key kp is visible to a query at qp iff
    kp <= qp (src/kernels.cuh:1416-1418; scripts/ref_engine.py:196-200), scores scaled by
    1/sqrt(D) (src/api.cu:600), query head h reads key/value head h // G
    (src/kernels.cuh:1347). `window` (not used by this architecture; the reference only guards
    it, src/api.cu:1296-1300) further hides keys with kp <= qp - window.
    q [T, Hq, D]; k, v [S, Hkv, D]; returns [T, Hq, D]."""
    T, Hq, D = q.shape
    Hkv = k.shape[1]
    G = Hq // Hkv
    kk, vv = k.repeat_interleave(G, 1), v.repeat_interleave(G, 1)
    scores = torch.einsum("thd,shd->hts", q, kk) / math.sqrt(D)
    qp = torch.as_tensor(q_pos)[:, None]
    kp = torch.as_tensor(k_pos)[None, :]
    visible = kp <= qp
    if window:
        visible = visible & (kp > qp - int(window))
    scores = scores.masked_fill(~visible[None], float("-inf"))
    p = torch.softmax(scores, -1)
    return torch.einsum("hts,shd->thd", p, vv)


def attention_block(xn, wq, wk, wv, wo, positions, n_heads, n_kv_heads, head_dim, inv_freq, window=None):
    """qkv projection, rotary on q and k (not v) after the projection, attention over the
    whole sequence, output projection (src/api.cu:1668-1691; scripts/ref_engine.py:175-201).
    Returns the block's output before the residual add."""
    T = xn.shape[0]
    q = (xn @ wq.T).reshape(T, n_heads, head_dim)
    k = (xn @ wk.T).reshape(T, n_kv_heads, head_dim)
    v = (xn @ wv.T).reshape(T, n_kv_heads, head_dim)
    cos, sin = rope_cos_sin(positions, inv_freq, xn.dtype)
    q, k = apply_rope(q, cos, sin), apply_rope(k, cos, sin)
    o = attention_scores_softmax_values(q, k, v, positions, positions, window)
    return o.reshape(T, n_heads * head_dim) @ wo.T


def swiglu_mlp(xn, wg, wu, wd):
    """act = silu(xn Wg^T) * (xn Wu^T) with silu(g) = g / (1 + exp(-g)); out = act Wd^T
    (src/kernels.cuh:100-105; src/api.cu:1708-1718; scripts/ref_engine.py:39-42, 213-215)."""
    g = xn @ wg.T
    u = xn @ wu.T
    return ((g / (1.0 + torch.exp(-g))) * u) @ wd.T


def lm_head(x, final_norm, w_head, eps):
    """logits = rmsnorm(x, final_norm) W^T, W the embedding table when tied
    (src/api.cu:1367, 1795-1812; scripts/ref_engine.py:232)."""
    return rmsnorm(x, final_norm, eps) @ w_head.T


# --------------------------------------------------------------------------------------
# whole model
# --------------------------------------------------------------------------------------
def forward(cfg, weights, tokens, positions=None, window=None):
    """Logits [T, vocab] of a whole token sequence: pre-norm blocks, x += attention(norm(x)),
    x += mlp(norm(x)) (scripts/ref_engine.py:218-232; src/api.cu:1728-1765)."""
    tokens = [int(t) for t in tokens]
    T = len(tokens)
    positions = list(range(T)) if positions is None else list(positions)
    D = head_dim_of(cfg)
    Hq, Hkv = cfg["num_attention_heads"], kv_heads_of(cfg)
    eps = cfg.get("rms_norm_eps", 1e-6)
    inv_freq = rope_inv_freq(D, cfg.get("rope_theta", 10000.0), cfg.get("rope_scaling"))
    x = embed(tokens, weights["model.embed_tokens.weight"])
    for l in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{l}."
        xn = rmsnorm(x, weights[p + "input_layernorm.weight"], eps)
        x = x + attention_block(xn, weights[p + "self_attn.q_proj.weight"], weights[p + "self_attn.k_proj.weight"],
                                weights[p + "self_attn.v_proj.weight"], weights[p + "self_attn.o_proj.weight"],
                                positions, Hq, Hkv, D, inv_freq, window)
        xn = rmsnorm(x, weights[p + "post_attention_layernorm.weight"], eps)
        x = x + swiglu_mlp(xn, weights[p + "mlp.gate_proj.weight"], weights[p + "mlp.up_proj.weight"],
                           weights[p + "mlp.down_proj.weight"])
    head = weights["model.embed_tokens.weight"] if cfg.get("tie_word_embeddings", False) else weights["lm_head.weight"]
    return lm_head(x, weights["model.norm.weight"], head, eps)


def argmax_lowest(logits):
    """Greedy choice: the largest value, the lowest index on ties, NaN above every number,
    index 0 when all are -inf (src/kernels.cuh:1883-1913)."""
    l = torch.as_tensor(logits, dtype=torch.float32)
    nan = torch.isnan(l)
    if bool(nan.any()):
        return int(torch.nonzero(nan)[0])
    best = l.max()
    return int(torch.nonzero(l == best)[0])


def generate_greedy(cfg, weights, prompt, n_new):
    """n_new greedy tokens, the first from the prompt's last logits
    (scripts/ref_engine.py:234-245), recomputing the whole sequence every time."""
    seq = [int(t) for t in prompt]
    out, steps = [], []
    for _ in range(n_new):
        logits = forward(cfg, weights, seq)[-1]
        steps.append(logits)
        t = argmax_lowest(logits)
        out.append(t)
        seq.append(t)
    return out, steps


# --------------------------------------------------------------------------------------
# temperature sampling (the reference is greedy only, README.md:94; this is the plain
# statement of what the engine's sampler has to do, with the same counter-based noise)
# --------------------------------------------------------------------------------------
def _mix32(x):
    """A 32-bit integer finaliser (xor-shift-multiply rounds) on Python ints."""
    x &= 0xFFFFFFFF
    x ^= x >> 16
    x = (x * 0x7FEB352D) & 0xFFFFFFFF
    x ^= x >> 15
    x = (x * 0x846CA68B) & 0xFFFFFFFF
    x ^= x >> 16
    return x


def sample_uniform(seed, position, index):
    """u in (0, 1) for (seed, position of the sampled token, vocabulary index): it depends on
    nothing else, so a draw is the same however the batch was put together."""
    h = _mix32((seed & 0xFFFFFFFF) ^ 0x9E3779B9)
    h = _mix32(h ^ ((position * 0x85EBCA6B) & 0xFFFFFFFF))
    h = _mix32(h ^ ((index * 0xC2B2AE35) & 0xFFFFFFFF))
    return ((h >> 8) + 0.5) / 16777216.0


def gumbel_scores(logits, temperature, seed, position):
    """logits / temperature + g, g = -log(-log u): the arg max of this is a draw from
    softmax(logits / temperature)."""
    l = torch.as_tensor(logits, dtype=torch.float64)
    u = torch.tensor([sample_uniform(seed, position, i) for i in range(l.numel())], dtype=torch.float64)
    return l / temperature - torch.log(-torch.log(u))


def sample_temperature(logits, temperature, seed, position):
    if temperature <= 0:
        return argmax_lowest(logits)
    return int(torch.argmax(gumbel_scores(logits, temperature, seed, position)))
