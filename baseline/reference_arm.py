"""The reference arm of bench.py: the UNMODIFIED Sky1219/hipinfer, built by its own Makefile line
for the GPU at hand and driven through its own Python binding (scripts/hipinfer.py), on the
same metric, sizes and workload as the engine's own arm. Nothing of hipinfer_b200 is imported here.

Build (`ensure_built`): Makefile, src/ and scripts/hipinfer.py are copied as they are from a
checkout of the reference into baseline/_ref/, and `make NV_ARCH="-gencode arch=compute_100,code=sm_100"`
runs there, which is what the reference's scripts/run_all.sh:63-68 does for a GPU whose arch
nvcc knows (Makefile:27-29 is the nvcc line). The binding loads the library named by
HIPINFER_LIB (scripts/hipinfer.py:7-8).

Weights: a random fp16 version-2 flat file at the asked shape, in the layout scripts/export.py:270-287
writes (64-byte header, inv_freq, embed, final norm, [head], per layer: norm, q/k/v stacked, o, norm,
gate/up interleaved by 16 rows, down; every tensor padded to 256 bytes).

Run: `Engine(path, max_batch, max_seq, max_prefill)`, `prefill(slot, ids)` for each slot,
`decode(B, warmup)`, then `decode(B, steps)`, whose return value is the GPU time of the steps
(CUDA graph path, scripts/hipinfer.py:423-424; src/api.cu decode_rank). The prefill figure is
the wall time of `prefill(0, ids)` (it returns the first token, so it has synchronised), as the
reference's own scripts/bench.py:377-383 takes it.
"""
from __future__ import annotations

import hashlib
import json
import math
import os
import shutil
import statistics
import struct
import subprocess
import sys
import tempfile
import time

HERE = os.path.dirname(os.path.abspath(__file__))
REF_DIR = os.path.join(HERE, "_ref")
REF_SRC = os.environ.get("HIPINFER_REFERENCE_SRC", "/root/reference")
NV_ARCH = "-gencode arch=compute_100,code=sm_100"
COPIED = ["Makefile", "src/api.cu", "src/kernels.cuh", "src/evict.cuh", "src/hip_compat.h", "scripts/hipinfer.py"]


class ReferenceUnavailable(RuntimeError):
    pass


def _digest(root: str) -> str:
    h = hashlib.sha256(NV_ARCH.encode())
    for rel in COPIED:
        with open(os.path.join(root, rel), "rb") as f:
            h.update(rel.encode() + b"\0" + f.read())
    return h.hexdigest()


def library_path() -> str:
    return os.path.join(REF_DIR, "build", "libhipinfer.so")


def ensure_built(verbose: bool = True) -> str:
    """Path of the reference's library, copying its sources and running its make line if need be."""
    so, stamp = library_path(), os.path.join(REF_DIR, "build", "stamp")
    have_copy = all(os.path.isfile(os.path.join(REF_DIR, rel)) for rel in COPIED)
    if os.path.isfile(so) and have_copy:
        try:
            if open(stamp).read().strip() == _digest(REF_DIR):
                return so
        except OSError:
            pass
        if not os.path.isdir(REF_SRC):
            return so        # built elsewhere and shipped: use it as it is
    if not os.path.isdir(REF_SRC):
        raise ReferenceUnavailable(f"no checkout of the reference at {REF_SRC} (HIPINFER_REFERENCE_SRC) and no built "
                                   f"library at {so}")
    for rel in COPIED:
        dst = os.path.join(REF_DIR, rel)
        os.makedirs(os.path.dirname(dst), exist_ok=True)
        shutil.copyfile(os.path.join(REF_SRC, rel), dst)
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.isfile(nvcc):
        raise ReferenceUnavailable("nvcc was not found: the reference's make line cannot run")
    if os.path.isfile(so):
        os.remove(so)
    if verbose:
        print(f"[reference] make in {REF_DIR} ({NV_ARCH}); this takes a few minutes", file=sys.stderr, flush=True)
    proc = subprocess.run(["make", f"NVCC={nvcc}", f"NV_ARCH={NV_ARCH}"], cwd=REF_DIR, stdout=subprocess.PIPE,
                          stderr=subprocess.STDOUT, text=True)
    if proc.returncode != 0 or not os.path.isfile(so):
        raise ReferenceUnavailable("the reference's make line failed: " + proc.stdout[-400:].replace("\n", " | "))
    with open(stamp, "w") as f:
        f.write(_digest(REF_DIR))
    return so


def llama3_inv_freq(head_dim: int, theta: float, scaling) -> list:
    """theta^(-2i/D), with the Llama-3 rule where `scaling` asks for it: frequencies whose wavelength is
    above original/low are divided by factor, those below original/high are kept, between them interpolated."""
    out = []
    for i in range(head_dim // 2):
        f = theta ** (-2.0 * i / head_dim)
        if scaling:
            orig = scaling["original_max_position_embeddings"]
            lo, hi, fac = scaling["low_freq_factor"], scaling["high_freq_factor"], scaling["factor"]
            wavelen = 2 * math.pi / f
            if wavelen > orig / lo:
                f = f / fac
            elif wavelen >= orig / hi:
                s = (orig / wavelen - lo) / (hi - lo)
                f = (1 - s) * f / fac + s * f
        out.append(f)
    return out


def write_random_weights(path: str, m: dict, layers: int, seed: int = 0, std: float = 0.02) -> int:
    """A random version-2 weight file for the model sizes `m` (HF config keys); returns its size."""
    import torch

    dev = "cuda" if torch.cuda.is_available() else "cpu"
    g = torch.Generator(device=dev).manual_seed(seed)
    V, H, I = m["vocab_size"], m["hidden_size"], m["intermediate_size"]
    Hq, Hkv, D = m["num_attention_heads"], m["num_key_value_heads"], m["head_dim"]
    tied = bool(m.get("tie_word_embeddings", False))
    head = struct.pack("<10i2f2i", 0x48495046, 2, V, H, I, layers, Hq, Hkv, D, m["max_position_embeddings"],
                       m["rms_norm_eps"], 1.0, 1 if tied else 0, 0)

    def pad(b: bytes) -> bytes:
        return b + b"\0" * (-len(b) % 256)

    def matrix(rows: int, cols: int) -> bytes:
        t = torch.randn(rows, cols, generator=g, device=dev, dtype=torch.float32).mul_(std).to(torch.float16)
        return pad(t.cpu().numpy().tobytes())

    def ones(n: int) -> bytes:
        return pad(torch.ones(n, dtype=torch.float16).numpy().tobytes())

    import numpy as np

    inv = np.asarray(llama3_inv_freq(D, m["rope_theta"], m.get("rope_scaling")), dtype=np.float32)
    with open(path, "wb") as f:
        f.write(head + b"\0" * (64 - len(head)))
        f.write(pad(inv.tobytes()))
        f.write(matrix(V, H))
        f.write(ones(H))
        if not tied:
            f.write(matrix(V, H))
        for _ in range(layers):
            f.write(ones(H))
            f.write(matrix((Hq + 2 * Hkv) * D, H))
            f.write(matrix(H, Hq * D))
            f.write(ones(H))
            f.write(matrix(2 * I, H))       # random rows: the interleaving of gate and up changes nothing
            f.write(matrix(H, I))
    return os.path.getsize(path)


def _prompts(n: int, length: int, vocab: int, seed: int):
    import torch

    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n, length), generator=g).tolist()


def run(model: dict, layers: int, batch: int, steps: int, warmup: int, context_len: int, prompt_len: int,
        prefill_tokens: int, point_batches=(), clock_sampler=None, tmp_root=None) -> dict:
    """Decode ms a step at `batch` (GPU time the engine reports), the same at `point_batches`, the
    wall time of a prefill and the end-to-end decode figure; raises ReferenceUnavailable."""
    import torch

    if not torch.cuda.is_available():
        raise ReferenceUnavailable("no CUDA device is visible")
    so = ensure_built()
    os.environ["HIPINFER_LIB"] = so
    sys.path.insert(0, os.path.join(REF_DIR, "scripts"))
    try:
        import hipinfer as hi
    except OSError as e:
        raise ReferenceUnavailable(f"the reference's library does not load: {e}") from None
    vocab = model["vocab_size"]
    max_batch = max([batch] + list(point_batches))
    with tempfile.TemporaryDirectory(dir=tmp_root) as tmp:
        path = os.path.join(tmp, "weights.bin")
        write_random_weights(path, model, layers)
        eng = hi.Engine(path, max_batch=max_batch, max_seq=context_len, max_prefill=max(prefill_tokens, prompt_len))

    def decode(B: int, n_steps: int, seed: int):
        ps = _prompts(B, prompt_len, vocab, seed)
        for b in range(B):
            eng.prefill(b, ps[b])
        eng.decode(B, warmup)                              # captures the graph of this batch size, warms up
        return eng.decode(B, n_steps) / n_steps            # GPU milliseconds

    out = {}
    if clock_sampler is not None:
        with clock_sampler:
            ms = decode(batch, steps, 1)
    else:
        ms = decode(batch, steps, 1)
    out["ms_per_step"] = ms
    out["points"] = {f"decode_b{batch}": batch / ms * 1e3}
    for b in point_batches:
        runs = [decode(b, min(steps, 64), 1) for _ in range(3)]
        out["points"][f"decode_b{b}"] = b / statistics.median(runs) * 1e3
    # prefill: one prompt in one call
    ids = _prompts(1, prefill_tokens, vocab, 3)[0]
    times = []
    for i in range(3 + 5):
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        eng.prefill(0, ids)
        times.append((time.perf_counter() - t0) * 1e3)
    out["prefill_ms"] = statistics.median(times[3:])
    # end to end: host tokens in (prefill), the decode call, and the produced tokens read back to the host
    n = min(steps, 64)
    ps = _prompts(batch, prompt_len, vocab, 2)
    for b in range(batch):
        eng.prefill(b, ps[b])
    eng.decode(batch, warmup)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    eng.decode(batch, n)
    toks = [eng.history(b, prompt_len + 1 + warmup, n) for b in range(batch)]
    out["e2e_ms_per_step"] = (time.perf_counter() - t0) * 1e3 / n
    assert all(len(t) == n for t in toks)
    out["weight_bytes"] = int(eng.weight_bytes)
    out["kv_bytes_per_token"] = int(eng.kv_bytes_per_token)
    eng.close()
    return out


if __name__ == "__main__":
    print(ensure_built())
