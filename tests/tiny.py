"""The tests' own small configurations (they differ in every size and option) and helpers to
make model folders with random weights in a temporary place and to replay traces."""
from __future__ import annotations

import json
import os
import subprocess
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

# 2 layers, 4/2 heads of 16, tied, plain rope, eps 1e-5
TINY_A = dict(architectures=["LlamaForCausalLM"], vocab_size=256, hidden_size=64, intermediate_size=128,
              num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=16,
              max_position_embeddings=128, rms_norm_eps=1e-5, rope_theta=10000.0, rope_scaling=None,
              tie_word_embeddings=True, hidden_act="silu")
# 3 layers, 3/1 heads of 32 (multi-query, group 3), untied, llama3 rope scaling, eps 1e-6, sizes no power of two
TINY_B = dict(architectures=["LlamaForCausalLM"], vocab_size=384, hidden_size=96, intermediate_size=320,
              num_hidden_layers=3, num_attention_heads=3, num_key_value_heads=1, head_dim=32,
              max_position_embeddings=256, rms_norm_eps=1e-6, rope_theta=500000.0,
              rope_scaling=dict(rope_type="llama3", factor=32.0, low_freq_factor=1.0, high_freq_factor=4.0,
                                original_max_position_embeddings=64),
              tie_word_embeddings=False, hidden_act="silu")
# a third one for the fast kernels' sizes: heads of 64, group 4, longer sequences, vocabulary no multiple of 64
TINY_C = dict(architectures=["LlamaForCausalLM"], vocab_size=1000, hidden_size=256, intermediate_size=704,
              num_hidden_layers=2, num_attention_heads=8, num_key_value_heads=2, head_dim=64,
              max_position_embeddings=1024, rms_norm_eps=1e-5, rope_theta=500000.0,
              rope_scaling=dict(rope_type="llama3", factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0,
                                original_max_position_embeddings=256),
              tie_word_embeddings=True, hidden_act="silu")

# sizes that the fast kernels take only in part: heads of 48 (the tensor-core attention kernels take 64 and 128), a width
# that is no multiple of 32, an odd vocabulary, multi-head attention without groups, one layer
TINY_D = dict(architectures=["LlamaForCausalLM"], vocab_size=515, hidden_size=200, intermediate_size=272,
              num_hidden_layers=1, num_attention_heads=5, num_key_value_heads=5, head_dim=48,
              max_position_embeddings=512, rms_norm_eps=3e-6, rope_theta=20000.0, rope_scaling=None,
              tie_word_embeddings=False, hidden_act="silu")
# heads of 80 in groups of 7, four layers, a width that is a multiple of 32 but not of 64
TINY_E = dict(architectures=["LlamaForCausalLM"], vocab_size=777, hidden_size=224, intermediate_size=400,
              num_hidden_layers=4, num_attention_heads=7, num_key_value_heads=1, head_dim=80,
              max_position_embeddings=512, rms_norm_eps=1e-5, rope_theta=1000000.0,
              rope_scaling=dict(rope_type="llama3", factor=4.0, low_freq_factor=1.0, high_freq_factor=4.0,
                                original_max_position_embeddings=128),
              tie_word_embeddings=True, hidden_act="silu")

# the real layer sizes of the Llama-3.2-1B shape (width, heads, feed-forward, vocabulary, llama3 scaling, tied head)
# with 2 of its 16 layers, so that the plain implementation on the CPU stays within seconds
LLAMA_1B_LAYERS_FULL, LLAMA_1B_LAYERS_TESTED = 16, 2
LLAMA_1B_2L = dict(architectures=["LlamaForCausalLM"], vocab_size=128256, hidden_size=2048, intermediate_size=8192,
                   num_hidden_layers=LLAMA_1B_LAYERS_TESTED, num_attention_heads=32, num_key_value_heads=8, head_dim=64,
                   max_position_embeddings=131072, rms_norm_eps=1e-5, rope_theta=500000.0,
                   rope_scaling=dict(rope_type="llama3", factor=32.0, low_freq_factor=1.0, high_freq_factor=4.0,
                                     original_max_position_embeddings=8192),
                   tie_word_embeddings=True, hidden_act="silu")

WEIGHTS = {"1b2l": dict(cfg=LLAMA_1B_2L, seed=11, std=0.02, norm_std=0.1),
           "a": dict(cfg=TINY_A, seed=0, std=0.02, norm_std=0.0),
           "b": dict(cfg=TINY_B, seed=2, std=0.05, norm_std=0.1),
           "c": dict(cfg=TINY_C, seed=5, std=0.04, norm_std=0.1),
           "d": dict(cfg=TINY_D, seed=6, std=0.05, norm_std=0.1),
           "e": dict(cfg=TINY_E, seed=8, std=0.04, norm_std=0.1)}


def make_model_folder(folder, which, dtype=torch.bfloat16):
    """config.json + model.safetensors of tiny model `which` through the product's own random-weights mode."""
    from hipinfer_b200.config import config_from_dict
    from hipinfer_b200.weights import write_random_model

    w = WEIGHTS[which]
    write_random_model(config_from_dict(w["cfg"]), str(folder), w["seed"], w["std"], w["norm_std"], dtype)
    return str(folder)


def random_tokens(n, vocab, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


class TraceRun:
    """bin/trace_run as a child process: send a step, wait for its `done` line, read its logits."""

    def __init__(self, model_dir, dtype, out_dir, max_tokens, extra=()):
        self.out_dir = str(out_dir)
        env = dict(os.environ)
        cmd = [sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", str(model_dir), "--dtype", dtype,
               "--out", self.out_dir, "--max-tokens", str(max_tokens)] + list(extra)
        self.p = subprocess.Popen(cmd, stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True, env=env)
        self.n = 0

    def step(self, entries, end=(), vocab=None):
        """entries: [(id, tokens, want)]. Returns float32 [wanted, vocab] or None."""
        rec = {"step": self.n, "entries": [{"id": i, "tokens": list(t), "want": list(w)} for i, t, w in entries],
               "end": list(end)}
        self.p.stdin.write(json.dumps(rec) + "\n")
        self.p.stdin.flush()
        while True:
            line = self.p.stdout.readline()
            if not line:
                raise RuntimeError(f"trace_run ended early (exit {self.p.wait()})")
            if line.strip() == f"done {self.n}":
                break
        path = os.path.join(self.out_dir, f"{self.n}.f32")
        self.n += 1
        nw = sum(len(w) for _, _, w in entries)
        if nw == 0:
            assert not os.path.exists(path)
            return None
        a = np.fromfile(path, dtype="<f4")
        return torch.from_numpy(a.reshape(nw, -1).copy())

    def close(self):
        self.p.stdin.close()
        rc = self.p.wait(timeout=120)
        assert rc == 0, f"trace_run exited with {rc}"


# ------------------------------------------------------------------------------------------
# cutting a set of requests into steps, and comparing all positions with the plain implementation
# ------------------------------------------------------------------------------------------
class RunnerStepper:
    """The same interface as TraceRun, straight on a ModelRunner in this process."""

    def __init__(self, runner):
        self.runner = runner

    def step(self, entries, end=()):
        from hipinfer_b200.engine import StepEntry

        logits = self.runner.step([StepEntry(i, t, w) for i, t, w in entries])
        for rid in end:
            self.runner.end(rid)
        return logits.float().cpu() if logits.shape[0] else None

    def close(self):
        pass


def plan_whole(requests):
    """Each request alone and whole."""
    return [[(rid, len(toks))] for rid, toks in requests.items()]


def plan_tail_decode(requests, tail=32):
    """Most of it in one step, the last `tail` tokens one by one."""
    plan = []
    for rid, toks in requests.items():
        head = max(1, len(toks) - tail)
        plan.append([(rid, head)])
        plan.extend([[(rid, 1)]] * (len(toks) - head))
    return plan


def plan_portions(requests, sizes=(7, 2, 16, 3, 2, 33, 5, 2, 64, 1, 9)):
    """Portions of changing size, down to two tokens."""
    plan = []
    for rid, toks in requests.items():
        left, i = len(toks), 0
        while left:
            n = min(sizes[i % len(sizes)], left)
            plan.append([(rid, n)])
            left -= n
            i += 1
    return plan


def plan_mixed(requests, seed=0, max_live=4, decode_tail=12):
    """Up to max_live live requests; prompt portions of some beside single decoded tokens of
    others; a request may sit out a step; requests end in another order than they started."""
    g = torch.Generator().manual_seed(seed)

    def rnd(lo, hi):
        return int(torch.randint(lo, hi + 1, (1,), generator=g))

    waiting = list(requests)
    left = {rid: len(t) for rid, t in requests.items()}
    live, plan = [], []
    while waiting or live:
        while waiting and len(live) < max_live and (not live or rnd(0, 2) > 0):
            live.append(waiting.pop(0))
        step = []
        for rid in list(live):
            if len(live) > 1 and rnd(0, 5) == 0:
                continue  # sits this step out
            n = 1 if left[rid] <= decode_tail else min(rnd(2, 19), left[rid] - decode_tail)
            step.append((rid, n))
            left[rid] -= n
            if left[rid] == 0:
                live.remove(rid)
        if step:
            plan.append(step)
    return plan


def plan_mixed_long(requests, seed=0, max_live=4, decode_tail=24, long=(65, 300), short=(2, 15)):
    """plan_mixed with the portions a scheduler with a budget of some hundred tokens makes: in a step one live
    request may take a long portion (more than 64 rows: the tensor-core products and the flash kernel over
    several key tiles, on top of what it has cached), the others short ones (2 to 15 rows) or, in their last
    `decode_tail` tokens, single rows. Requests sit out steps and end in another order than they started."""
    g = torch.Generator().manual_seed(1000 + seed)

    def rnd(lo, hi):
        return int(torch.randint(lo, hi + 1, (1,), generator=g))

    waiting = list(requests)
    left = {rid: len(t) for rid, t in requests.items()}
    live, plan = [], []
    while waiting or live:
        while waiting and len(live) < max_live and (not live or rnd(0, 2) > 0):
            live.append(waiting.pop(0))
        step, long_taken = [], False
        for rid in sorted(live, key=lambda r: -left[r]):       # the request with most left gets the long portion
            if len(live) > 1 and rnd(0, 6) == 0:
                continue  # sits this step out
            room = left[rid] - decode_tail
            if room <= 0:
                n = 1
            elif not long_taken and room > short[1] and rnd(0, 3) > 0:
                n, long_taken = min(rnd(*long), room), True
            else:
                n = min(rnd(*short), room)
            step.append((rid, n))
            left[rid] -= n
            if left[rid] == 0:
                live.remove(rid)
        if step:
            step.sort(key=lambda e: list(requests).index(e[0]))
            plan.append(step)
    return plan


def run_plan(stepper, requests, plan):
    """Feed `plan` (steps of (id, n tokens)) wanting every position; {id: logits [len, vocab]}."""
    fed = {rid: 0 for rid in requests}
    out = {rid: [] for rid in requests}
    for step in plan:
        entries, end = [], []
        for rid, n in step:
            toks = requests[rid][fed[rid]:fed[rid] + n]
            entries.append((rid, toks, list(range(n))))
            fed[rid] += n
            if fed[rid] == len(requests[rid]):
                end.append(rid)
        logits = stepper.step(entries, end)
        o = 0
        for rid, n in step:
            out[rid].append(logits[o:o + n])
            o += n
    assert all(fed[r] == len(requests[r]) for r in requests)
    return {rid: torch.cat(v) for rid, v in out.items()}


# Tolerances, as a fraction of the largest |logit| of the request. 32-bit: rounding of sums in
# another order. bfloat16: activations, q, k, v and the attention output are rounded to 8 bits
# of mantissa a few times per layer. The bounds stand about a factor of two above what the
# engine measures (printed at the end of every run): 32-bit 2.5e-7 (tiny A) to 4.2e-6 (1B layer
# sizes, 2 layers); bfloat16 2.1e-3 (tiny A) to 8.8e-3 (tiny B and the 1B layer sizes). They are
# meant for these models of two and three layers: the error grows with depth. That the same
# step function holds 4e-6 in 32-bit under every cutting is what rules out a fault of the cache
# or the batch hiding below the bfloat16 bound.
TOL = {"float32": 1e-5, "bfloat16": 1.5e-2}
MEASURED = []      # ((configuration, plan), dtype, largest |difference| / largest |logit|) of every comparison: printed at the end of a run


def assert_logits_close(got, ref, dtype, what="", group=None):
    """group: (configuration, plan) under which the measured error is listed at the end of the run."""
    scale = float(ref.abs().max())
    err = float((got.float() - ref.float()).abs().max())
    assert got.shape == ref.shape, f"{what}: shape {tuple(got.shape)} != {tuple(ref.shape)}"
    assert torch.isfinite(got).all(), f"{what}: non-finite logits"
    MEASURED.append((group or (what, ""), dtype, err / scale if scale else 0.0))
    if err > TOL[dtype] * scale:
        bad = (got.float() - ref.float()).abs().amax(-1)
        first = int((bad > TOL[dtype] * scale).nonzero()[0])
        raise AssertionError(f"{what}: max |diff| {err:.3e} > {TOL[dtype]:.0e} * {scale:.3e}; first wrong "
                             f"position {first} of {got.shape[0]} (diff there {float(bad[first]):.3e})")
    return err / scale
