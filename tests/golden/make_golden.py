"""Makes the committed anchors `tiny_a.npz` and `tiny_b.npz`.

It runs Sky1219/hipinfer's own CPU oracle, `scripts/ref_engine.py` in its never-rounding mode
"fp32", on two tiny random dense models and stores the logits. `tests/test_plain.py` rebuilds
the same weights with `golden_weights()` below and compares `tests/plain_llama.py` with the
stored logits. The oracle reads the project's flat weight file (version 2: a 64-byte header,
then tensors in a fixed order, each padded to 256 bytes, fp16 values; scripts/export.py:5-17,
scripts/ref_engine.py:93-135), so this script writes such a file from the weights first: q, k, v
stacked by rows, gate and up interleaved in groups of 16 rows (scripts/export.py:97-101, 278).
`inv_freq` is data in that file (scripts/export.py:104-108): for the model with Llama-3
frequency scaling it is computed by the plain implementation, so the scaling formula itself is
not anchored by the oracle, only its use.

    python tests/golden/make_golden.py --reference /path/to/hipinfer

Needs numpy and torch on the CPU only. The weights come from an integer hash, not from a
library's random generator, so that they are the same everywhere.
"""
from __future__ import annotations

import argparse
import os
import struct
import sys
import tempfile

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))

GOLDEN = {
    "tiny_a": dict(
        cfg=dict(architectures=["LlamaForCausalLM"], vocab_size=256, hidden_size=64, intermediate_size=128,
                 num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=16,
                 max_position_embeddings=128, rms_norm_eps=1e-5, rope_theta=10000.0, rope_scaling=None,
                 tie_word_embeddings=True, hidden_act="silu"),
        seed=11, n_tokens=17, norm_noise=False),
    "tiny_b": dict(
        cfg=dict(architectures=["LlamaForCausalLM"], vocab_size=384, hidden_size=96, intermediate_size=320,
                 num_hidden_layers=3, num_attention_heads=3, num_key_value_heads=1, head_dim=32,
                 max_position_embeddings=256, rms_norm_eps=1e-6, rope_theta=500000.0,
                 rope_scaling=dict(rope_type="llama3", factor=32.0, low_freq_factor=1.0, high_freq_factor=4.0,
                                   original_max_position_embeddings=64),
                 tie_word_embeddings=False, hidden_act="silu"),
        seed=23, n_tokens=24, norm_noise=True),
}


def _hash_u32(n, seed):
    """n 32-bit hashes of 0..n-1 under `seed` (xor-shift-multiply rounds on uint64 lanes)."""
    x = (np.arange(n, dtype=np.uint64) + np.uint64(seed) * np.uint64(0x9E3779B1)) & np.uint64(0xFFFFFFFF)
    for mul, sh in ((0x7FEB352D, 15), (0x846CA68B, 16)):
        x ^= x >> np.uint64(16)
        x = (x * np.uint64(mul)) & np.uint64(0xFFFFFFFF)
        x ^= x >> np.uint64(sh)
    return x


def _matrix(shape, seed):
    """Values k * 2^-15, k in [-2048, 2048): exact in fp16, spread over about +-0.06."""
    n = int(np.prod(shape))
    k = (_hash_u32(n, seed) % np.uint64(4096)).astype(np.int64) - 2048
    return torch.from_numpy((k.astype(np.float64) * 2.0 ** -15).astype(np.float32).reshape(shape))


def _norm(n, seed, noise):
    if not noise:
        return torch.ones(n)
    k = (_hash_u32(n, seed) % np.uint64(256)).astype(np.int64) - 128
    return torch.from_numpy((1.0 + k.astype(np.float64) * 2.0 ** -10).astype(np.float32))


def golden_weights(name):
    """{HF tensor name: float32 tensor} of one golden model; every value is exact in fp16."""
    g = GOLDEN[name]
    c, seed = g["cfg"], g["seed"]
    H, I, V, D = c["hidden_size"], c["intermediate_size"], c["vocab_size"], c["head_dim"]
    Hq, Hkv = c["num_attention_heads"], c["num_key_value_heads"]
    w, s = {}, seed * 1000
    w["model.embed_tokens.weight"] = _matrix((V, H), s + 1)
    w["model.norm.weight"] = _norm(H, s + 2, g["norm_noise"])
    if not c["tie_word_embeddings"]:
        w["lm_head.weight"] = _matrix((V, H), s + 3)
    for l in range(c["num_hidden_layers"]):
        p, b = f"model.layers.{l}.", s + 10 * (l + 1)
        w[p + "input_layernorm.weight"] = _norm(H, b, g["norm_noise"])
        w[p + "self_attn.q_proj.weight"] = _matrix((Hq * D, H), b + 1)
        w[p + "self_attn.k_proj.weight"] = _matrix((Hkv * D, H), b + 2)
        w[p + "self_attn.v_proj.weight"] = _matrix((Hkv * D, H), b + 3)
        w[p + "self_attn.o_proj.weight"] = _matrix((H, Hq * D), b + 4)
        w[p + "post_attention_layernorm.weight"] = _norm(H, b + 5, g["norm_noise"])
        w[p + "mlp.gate_proj.weight"] = _matrix((I, H), b + 6)
        w[p + "mlp.up_proj.weight"] = _matrix((I, H), b + 7)
        w[p + "mlp.down_proj.weight"] = _matrix((H, I), b + 8)
    return w


def golden_tokens(name):
    g = GOLDEN[name]
    return [int(t) for t in _hash_u32(g["n_tokens"], g["seed"] + 7) % np.uint64(g["cfg"]["vocab_size"])]


def write_flat_file(path, name):
    """The reference's version-2 weight file for one golden model."""
    import plain_llama as plain

    g = GOLDEN[name]
    c, w = g["cfg"], golden_weights(name)
    D = c["head_dim"]
    inv = plain.rope_inv_freq(D, c["rope_theta"], c["rope_scaling"]).numpy().astype(np.float32)
    flags = 1 if c["tie_word_embeddings"] else 0
    head = struct.pack("<10i2f2i", 0x48495046, 2, c["vocab_size"], c["hidden_size"], c["intermediate_size"],
                       c["num_hidden_layers"], c["num_attention_heads"], c["num_key_value_heads"], D,
                       c["max_position_embeddings"], c["rms_norm_eps"], 1.0, flags, 0)

    def pad(b):
        return b + b"\0" * (-len(b) % 256)

    def f16(t):
        a = t.numpy().astype(np.float16)
        assert np.array_equal(a.astype(np.float32), t.numpy()), "golden weights must be exact in fp16"
        return pad(a.tobytes())

    with open(path, "wb") as f:
        f.write(head + b"\0" * (64 - len(head)))
        f.write(pad(inv.tobytes()))
        f.write(f16(w["model.embed_tokens.weight"]))
        f.write(f16(w["model.norm.weight"]))
        if not c["tie_word_embeddings"]:
            f.write(f16(w["lm_head.weight"]))
        for l in range(c["num_hidden_layers"]):
            p = f"model.layers.{l}."
            f.write(f16(w[p + "input_layernorm.weight"]))
            f.write(f16(torch.cat([w[p + "self_attn.q_proj.weight"], w[p + "self_attn.k_proj.weight"],
                                   w[p + "self_attn.v_proj.weight"]])))
            f.write(f16(w[p + "self_attn.o_proj.weight"]))
            f.write(f16(w[p + "post_attention_layernorm.weight"]))
            gate, up = w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"]
            I, H = gate.shape
            gu = torch.stack([gate.reshape(I // 16, 16, H), up.reshape(I // 16, 16, H)], 1).reshape(2 * I, H)
            f.write(f16(gu))
            f.write(f16(w[p + "mlp.down_proj.weight"]))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="checkout of Sky1219/hipinfer")
    a = ap.parse_args()
    sys.path.insert(0, os.path.join(a.reference, "scripts"))
    import ref_engine

    for name in GOLDEN:
        with tempfile.TemporaryDirectory() as tmp:
            path = os.path.join(tmp, name + ".bin")
            write_flat_file(path, name)
            eng = ref_engine.RefEngine(path, "fp32")
            tokens = golden_tokens(name)
            whole = eng.forward(tokens).numpy().astype(np.float32)
            eng.reset()
            stepwise = np.concatenate([eng.forward([t]).numpy() for t in tokens]).astype(np.float32)
        print(name, whole.shape, "whole vs token by token:", float(np.abs(whole - stepwise).max()))
        np.savez(os.path.join(HERE, name + ".npz"), tokens=np.array(tokens, dtype=np.int32), logits=whole)


if __name__ == "__main__":
    main()
