#!/usr/bin/env python3
"""Decode and prefill throughput of hipinfer_b200 at Llama-3.2-1B shape with random weights.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--batch 8] [--layers L] [--impl ours|reference]
                    [--shape 1b|3b|8b] [--prompt N] [--prefill-tokens N]      (further sizes; the default is 1b, 2048, 2048)

One JSON line on stdout. `value` is decoded tokens a second at the given batch: K decode steps
(forward from the paged cache + on-device sampling, the sampled tokens feeding the next step on
the device) timed with CUDA events after W warm-up steps; the requests hold 2,048-token random
prompts, so the steps run at contexts 2,048 + W .. 2,048 + W + K. `e2e` is the same through
`Engine.step()` (scheduler, host tokens in and out). `prefill` is one 2,048-token prompt in one
step. `roofline` divides the bytes a decode step has to read (every weight it uses once, and the
cache of the live requests) by its time. Peaks come from MEASURED_PEAKS.json beside this file,
else from the fallback figures. The batch-1 and batch-64 points are the median of three runs of
64 steps each. The reference measures the same quantities in
scripts/bench.py:384-449 (decode over many replayed steps, floor = weight + cache bytes / peak).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# the default run: Llama-3.2-1B shape
MODEL = dict(architectures=["LlamaForCausalLM"], vocab_size=128256, hidden_size=2048, intermediate_size=8192,
             num_hidden_layers=16, num_attention_heads=32, num_key_value_heads=8, head_dim=64,
             max_position_embeddings=131072, rms_norm_eps=1e-5, rope_theta=500000.0,
             rope_scaling=dict(rope_type="llama3", factor=32.0, low_freq_factor=1.0, high_freq_factor=4.0,
                               original_max_position_embeddings=8192),
             tie_word_embeddings=True, hidden_act="silu")
CONTEXT_LEN, PROMPT_LEN, PREFILL_TOKENS, PAGE = 4096, 2048, 2048, 16
# further layer shapes of the same architecture for --shape (Llama-3.2-3B and Llama-3.1-8B sizes)
SHAPES = {
    "1b": dict(name="Llama-3.2-1B shape"),
    "3b": dict(name="Llama-3.2-3B shape", hidden_size=3072, intermediate_size=8192, num_hidden_layers=28,
               num_attention_heads=24, num_key_value_heads=8, head_dim=128, tie_word_embeddings=True),
    "8b": dict(name="Llama-3.1-8B shape", hidden_size=4096, intermediate_size=14336, num_hidden_layers=32,
               num_attention_heads=32, num_key_value_heads=8, head_dim=128, tie_word_embeddings=False, rope_factor=8.0),
}
SHAPE_NAME = SHAPES["1b"]["name"]


def choose_shape(shape: str, prompt_len: int, prefill_tokens: int, steps: int) -> None:
    """Other sizes than the default run: the layer shape, the length of the prompts behind the
    decode steps and the length of the prefill. The context length grows with them."""
    global SHAPE_NAME, CONTEXT_LEN, PROMPT_LEN, PREFILL_TOKENS
    spec = dict(SHAPES[shape])
    SHAPE_NAME = spec.pop("name")
    factor = spec.pop("rope_factor", None)
    MODEL.update(spec)
    if factor is not None:
        MODEL["rope_scaling"] = dict(MODEL["rope_scaling"], factor=factor)
    PROMPT_LEN, PREFILL_TOKENS = prompt_len, prefill_tokens
    CONTEXT_LEN = max(CONTEXT_LEN, -(-(max(prompt_len, prefill_tokens) + steps + 256) // 1024) * 1024)
FALLBACK_PEAKS = dict(hbm_gbs=6650.0, bf16_tflops=1590.0, bf16_tflops_sustained=1400.0)


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(p):
        with open(p) as f:
            d = json.load(f)
        return dict(hbm_gbs=float(d["hbm_gbs"]), bf16_tflops=float(d["bf16_tflops"]),
                    bf16_tflops_sustained=float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), source="measured")
    return dict(FALLBACK_PEAKS, source="fallback")


class ClockSampler:
    """nvidia-smi clocks and throttle reasons while the timed region runs (reading only). The
    process is started ahead of the region (it takes a while to print its first line); only the
    lines that arrive between `with` entry and exit count."""

    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.rows, self.proc, self.t0, self.t1 = [], None, None, None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "20"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.monotonic(), [c.strip() for c in line.split(",")]))

    def __enter__(self):
        if self.proc is None:
            self.start()
        self.t0 = time.monotonic()
        return self

    def __exit__(self, *a):
        self.t1 = time.monotonic()
        if self.proc:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self):
        rows = [r for t, r in self.rows if self.t0 is not None and self.t0 <= t <= self.t1 + 0.02 and len(r) >= 6]
        sm = [int(r[0]) for r in rows if r[0].isdigit()]
        mx = [int(r[1]) for r in rows if r[1].isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(r[2 + i].lower().startswith("active") for r in rows)]
        return dict(sm_mhz=int(statistics.median(sm)) if sm else None, sm_max_mhz=max(mx) if mx else None,
                    reasons=reasons, samples=len(sm))


def build_engine(layers: int, max_batch: int, total_steps: int):
    import torch  # noqa: F401
    from hipinfer_b200 import Engine

    cfg = dict(MODEL, num_hidden_layers=layers)
    pages_per_seq = -(-(PROMPT_LEN + total_steps + 2 * max_batch + 4 * PAGE) // PAGE)
    num_pages = max(max_batch * pages_per_seq, -(-PREFILL_TOKENS // PAGE)) + 8
    return Engine(config=cfg, random_weights=0, std=0.02, dtype="bfloat16", max_batch=max_batch, max_seq=CONTEXT_LEN,
                  max_prefill=max(PREFILL_TOKENS, PROMPT_LEN), page_size=PAGE, num_pages=num_pages)


def prompts(n, seed, length=None):
    import torch

    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, MODEL["vocab_size"], (n, length or PROMPT_LEN), generator=g).tolist()


def decode_device(eng, batch: int, steps: int, warmup: int, sampler=None):
    """K decode steps timed on the device; the sampled tokens stay on the device. Returns
    (ms per step, mean context of the timed steps, launches per step)."""
    import torch

    from hipinfer_b200.engine import StepEntry
    from hipinfer_b200.kernels import library, ops

    runner = eng.runner
    ids = [("bench", batch, i) for i in range(batch)]
    first = []
    for rid, p in zip(ids, prompts(batch, 1)):
        logits = runner.step([StepEntry(rid, p, [PROMPT_LEN - 1])])
        first.append(ops.sample(logits, None, None, None))
    tokens = torch.cat(first).contiguous()
    entries = [StepEntry(rid, [0], [0]) for rid in ids]

    def one():
        logits = runner.step(entries, device_tokens=tokens)
        ops.sample(logits, None, None, None, out=tokens)

    for _ in range(warmup):
        one()
    torch.cuda.synchronize()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    l0 = library.launches[0]
    with (sampler or _Null()):
        start.record()
        for _ in range(steps):
            one()
        stop.record()
        stop.synchronize()
    ms = start.elapsed_time(stop) / steps
    launches = (library.launches[0] - l0) / steps
    from hipinfer_b200.kernels import fast
    fast.check_status()
    for rid in ids:
        runner.end(rid)
    return ms, PROMPT_LEN + warmup + (steps - 1) / 2.0 + 1, launches


class _Null:
    def __enter__(self):
        return self

    def __exit__(self, *a):
        pass


def decode_e2e(eng, batch: int, steps: int, warmup: int):
    """The same through Engine.step(): scheduler, batch built on the host and copied from pinned
    memory every step, sampled tokens read back every step. Wall clock around synchronised ends."""
    import torch

    # requests that finish their prompt early decode while the others are still being prefilled
    # (at most 2 * batch steps): leave enough tokens that nobody finishes inside the timed steps
    for p in prompts(batch, 2):
        eng.add_request(p, warmup + steps + 2 * batch + 8)
    while any(not r.decoding for r in eng.scheduler.running) or eng.scheduler.waiting:
        eng.step()
    for _ in range(warmup):
        eng.step()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(steps - 1):
        eng.step()
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    assert len(eng.scheduler.running) == batch, "a request finished inside the timed steps"
    eng.abort_all()                                # the measurement is over: drop the requests
    groups = len(eng.runner.cache.groups)
    width = -(-CONTEXT_LEN // PAGE)
    n_int = 4 * batch + 4 * batch + batch + groups * batch * width + groups * batch
    return dt / (steps - 1) * 1e3, n_int * 4, batch * 4


def prefill_device(eng, warmup: int, reps: int):
    import torch

    from hipinfer_b200.engine import StepEntry
    from hipinfer_b200.kernels import fast

    runner = eng.runner
    toks = prompts(1, 3, PREFILL_TOKENS)[0]
    times = []
    for i in range(warmup + reps):
        torch.cuda.synchronize()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        runner.step([StepEntry(("prefill", i), toks, [PREFILL_TOKENS - 1])])
        stop.record()
        stop.synchronize()
        runner.end(("prefill", i))
        if i >= warmup:
            times.append(start.elapsed_time(stop))
    fast.check_status()
    return statistics.median(times)


def self_check(eng, tail: int = 8):
    """What the timed steps compute, checked at the benchmark's own sizes: the logits of the last `tail` positions of a
    short request, once from decode steps over the cache (graph replay, the timed path) and once from a single step
    over the whole request (the prefill path, which the tests compare with the plain implementation at these layer
    sizes). Returns (all finite, largest |difference| / largest |logit|, smallest cosine between a position's two rows
    of logits)."""
    import torch

    from hipinfer_b200.engine import StepEntry

    runner = eng.runner
    n = 160
    toks = prompts(1, 5, n)[0]
    whole = runner.step([StepEntry("check-whole", toks, list(range(n - tail, n)))]).float()
    runner.end("check-whole")
    runner.step([StepEntry("check-steps", toks[:n - tail], [])])
    rows = [runner.step([StepEntry("check-steps", [t], [0])]).float().clone() for t in toks[n - tail:]]
    runner.end("check-steps")
    steps = torch.cat(rows)
    finite = bool(torch.isfinite(whole).all()) and bool(torch.isfinite(steps).all()) and float(whole.abs().max()) > 0
    drift = float((whole - steps).abs().max()) / max(float(whole.abs().max()), 1e-30)
    cosine = float(torch.nn.functional.cosine_similarity(whole, steps, dim=-1).min()) if finite else 0.0
    return finite, drift, cosine


def mixed_workload(a) -> int:
    """The scheduler's own workload: `--requests` requests with
    uniform-random prompt lengths in [64, 2048] (seeded), prompts cut into portions under a budget of
    `--max-prefill` tokens a step beside the decode rows of the others, `--new` tokens each, through
    Engine.add_request / Engine.step. One JSON line: generated and processed tokens a second over the whole
    run (wall clock around synchronised ends, host tokens in and out), the device time of the same region
    (CUDA events), steps split into those that carry prompt portions and decode-only ones, preemptions."""
    import torch

    from hipinfer_b200 import Engine

    layers = a.layers or MODEL["num_hidden_layers"]
    g = torch.Generator().manual_seed(7)
    lens = torch.randint(64, 2049, (a.requests,), generator=g).tolist()
    ps = [torch.randint(0, MODEL["vocab_size"], (n,), generator=g).tolist() for n in lens]
    max_seq = 2048 + a.new + 64
    pages = a.requests * -(-(2048 + a.new) // PAGE) + 8
    if a.pool_fraction < 1.0:
        pages = max(int(pages * a.pool_fraction), -(-(2048 + a.new) // PAGE) + 8)
    eng = Engine(config=dict(MODEL, num_hidden_layers=layers), random_weights=0, std=0.02, dtype="bfloat16",
                 max_batch=a.requests, max_seq=max_seq, max_prefill=a.max_prefill, page_size=PAGE, num_pages=pages)

    def run_once(timed):
        for p in ps:
            eng.add_request(p, a.new)
        kinds = {"prefill": [0, 0.0, 0], "decode": [0, 0.0, 0]}
        torch.cuda.synchronize()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        t0 = time.perf_counter()
        n_done, host = 0, 0.0
        while eng.scheduler.has_work() or eng._pending is not None or eng._unreported:
            h0 = time.perf_counter()
            n_done += len(eng.step())
            dt = time.perf_counter() - h0
            host += dt
            if eng.last_step is not None:
                k = kinds["prefill" if eng.last_step[2] else "decode"]
                k[0] += 1
                k[1] += dt
                k[2] += eng.last_step[0]
        stop.record()
        stop.synchronize()
        wall = time.perf_counter() - t0
        assert n_done == a.requests
        return wall, start.elapsed_time(stop) / 1e3, kinds

    run_once(False)                       # warm-up: compiles nothing new afterwards, graphs of the decode sizes captured
    pre0 = eng.scheduler.n_preemptions
    clocks = ClockSampler().start()
    with clocks:
        wall, dev, kinds = run_once(True)
    from hipinfer_b200.kernels import ops
    ops.check_device_status()
    gen = a.requests * a.new
    total = sum(lens) + gen - a.requests
    steps = kinds["prefill"][0] + kinds["decode"][0]
    out = {
        "metric": f"mixed workload, generated tok/s ({SHAPE_NAME}: {a.requests} requests, prompts U[64, 2048], "
                  f"{a.max_prefill}-token budget, {a.new} new tokens each)",
        "value": round(gen / wall, 1), "unit": "tok/s", "n_gpus": 1, "steps": steps, "warmup": 1,
        "ms_per_step": round(wall / steps * 1e3, 4), "higher_is_better": True, "dtype": "bf16", "impl": "ours",
        "data": "synthetic: uniform-random token ids and prompt lengths (seed 7), random N(0, 0.02) bf16 weights",
        "config": dict(bench_config(a.requests, layers, "inputs larger than L2"), max_prefill=a.max_prefill, new_tokens=a.new,
                       prompt_tokens=sum(lens), pool_pages=pages),
        "processed_tok_s": round(total / wall, 1), "wall_s": round(wall, 4), "device_s": round(dev, 4),
        "e2e_over_device": round(wall / dev, 4),
        "steps_with_prompt_portions": {"steps": kinds["prefill"][0], "rows": kinds["prefill"][2],
                                       "host_ms_per_step": round(kinds["prefill"][1] / max(1, kinds["prefill"][0]) * 1e3, 4)},
        "decode_only_steps": {"steps": kinds["decode"][0], "rows": kinds["decode"][2],
                              "host_ms_per_step": round(kinds["decode"][1] / max(1, kinds["decode"][0]) * 1e3, 4)},
        "preemptions": eng.scheduler.n_preemptions - pre0, "clocks": clocks.summary(),
    }
    eng.close()
    print(json.dumps(out))
    return 0


def prefill_flops(layers: int) -> float:
    m, T = MODEL, PREFILL_TOKENS
    H, I, D, Hq, Hkv, V = (m["hidden_size"], m["intermediate_size"], m["head_dim"], m["num_attention_heads"],
                           m["num_key_value_heads"], m["vocab_size"])
    per_layer = (Hq + 2 * Hkv) * D * H + H * Hq * D + 3 * I * H
    linear = 2.0 * T * per_layer * layers
    attention = 4.0 * Hq * D * (T * (T + 1) / 2) * layers   # causal: q k^T and p v over the visible keys
    return linear + attention + 2.0 * V * H


def breakdown(layers: int, batch: int, prefill: bool = False) -> int:
    """With prefill: the same for one prefill step of PREFILL_TOKENS tokens (not graph-replayed). Otherwise:
    the time line of one graph-replayed decode step at `batch` from torch's CUPTI profiler (a
    table on stdout, not the JSON line). Kernels overlap (programmatic dependent launch: they start
    early and wait), so besides start and duration the table gives, for the kernels of one layer in
    the middle of the step, the time from the end of the kernel before to the kernel's own end: its
    share of the chain. Below it the kernels by name with their summed durations."""
    import json as _json
    import tempfile

    import torch
    from torch.profiler import ProfilerActivity, profile

    from hipinfer_b200.engine import StepEntry
    from hipinfer_b200.kernels import ops

    eng = build_engine(layers, max(batch, 2), 64)
    runner = eng.runner
    if prefill:
        toks, count = prompts(1, 3, PREFILL_TOKENS)[0], [0]

        def one():
            count[0] += 1
            runner.step([StepEntry(("bd", count[0]), toks, [PREFILL_TOKENS - 1])])
            runner.end(("bd", count[0]))
    else:
        ids = [("bd", i) for i in range(batch)]
        first = [ops.sample(runner.step([StepEntry(rid, p, [PROMPT_LEN - 1])]), None, None, None)
                 for rid, p in zip(ids, prompts(batch, 1))]
        tokens = torch.cat(first).contiguous()
        entries = [StepEntry(rid, [0], [0]) for rid in ids]

        def one():
            ops.sample(runner.step(entries, device_tokens=tokens), None, None, None, out=tokens)

    for _ in range(5):
        one()
    torch.cuda.synchronize()
    n = 4
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        for _ in range(n):
            one()
        torch.cuda.synchronize()
    with tempfile.TemporaryDirectory() as tmp:
        path = os.path.join(tmp, "trace.json")
        prof.export_chrome_trace(path)
        with open(path) as f:
            events = [e for e in _json.load(f)["traceEvents"] if e.get("cat") == "kernel"]
    events.sort(key=lambda e: e["ts"])
    per = len(events) // n
    step = events[2 * per: 3 * per]                      # the third of the four steps
    t0 = step[0]["ts"]
    span = step[-1]["ts"] + step[-1]["dur"] - t0
    what = f"prefill step of {PREFILL_TOKENS} tokens" if prefill else f"decode step at batch {batch}, context {PROMPT_LEN}+"
    print(f"{what}: {per} kernels, {span:.1f} us from the first kernel's start to the last one's end")
    # besides the layers: embedding, last norm, head, and in a decode step the sampling kernel
    per_layer = max(1, (per - (3 if prefill else 4)) // max(1, layers))
    lo = min(len(step) - 1, 1 + per_layer * (layers // 2))
    print(f"kernels {lo}..{lo + per_layer - 1} (one layer): start, duration, end minus the end of the kernel before")
    prev_end = max(e["ts"] + e["dur"] for e in step[:lo]) if lo else t0
    for e in step[lo: lo + per_layer]:
        end = e["ts"] + e["dur"]
        print(f"{e['ts'] - t0:9.2f} us  dur {e['dur']:7.2f}  chain {end - prev_end:6.2f}  {e['name'][:56]:56s} grid {e['args'].get('grid')}")
        prev_end = max(prev_end, end)
    agg = {}
    for e in step:
        a = agg.setdefault(e["name"][:70], [0, 0.0])
        a[0] += 1
        a[1] += e["dur"]
    print("by kernel (durations overlap and do not add up to the step):")
    for name, (cnt, us) in sorted(agg.items(), key=lambda kv: -kv[1][1]):
        print(f"{us:9.1f} us  {cnt:4d} launches  {us / cnt:7.2f} us each  {name}")
    eng.close()
    return 0


def reference_arm(a) -> int:
    """The unmodified reference through its own binding (baseline/reference_arm.py builds it with its
    own make line and drives `Engine.prefill` / `Engine.decode`): the same metric, sizes, steps and
    warm-up as the other arm, fp16 as the reference computes. Nothing of hipinfer_b200 is imported."""
    sys.path.insert(0, os.path.join(ROOT, "baseline"))
    import reference_arm as ra

    if a.gpus != 1:
        print(json.dumps({"impl": "reference", "unavailable": "this bench compares on one GPU"}))
        return 0
    a.warmup = max(a.warmup, 3)
    if (a.shape, a.prompt, a.prefill_tokens) != ("1b", PROMPT_LEN, PREFILL_TOKENS):
        choose_shape(a.shape, a.prompt, a.prefill_tokens, a.steps + a.warmup + 8)
    layers = a.layers or MODEL["num_hidden_layers"]
    point_batches = [] if a.no_points else [b for b in (1, 64) if b != a.batch]
    clocks = ClockSampler().start()
    try:
        r = ra.run(MODEL, layers, a.batch, a.steps, a.warmup, CONTEXT_LEN, PROMPT_LEN, PREFILL_TOKENS, point_batches, clocks)
    except ra.ReferenceUnavailable as e:
        print(json.dumps({"impl": "reference", "unavailable": str(e)}))
        return 0
    pk = peaks()
    ms = r["ms_per_step"]
    mean_ctx = PROMPT_LEN + a.warmup + (a.steps - 1) / 2.0 + 1
    step_bytes = r["weight_bytes"] + a.batch * mean_ctx * r["kv_bytes_per_token"]
    achieved = step_bytes / ms / 1e6
    pre_ms = r["prefill_ms"]
    out = {
        "metric": f"decode tok/s at batch {a.batch} ({SHAPE_NAME}, {PROMPT_LEN:,}-token prompts)",
        "value": round(a.batch / ms * 1e3, 1), "unit": "tok/s", "n_gpus": 1, "steps": a.steps, "warmup": a.warmup,
        "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "fp16", "data": "synthetic: uniform-random token ids, random N(0, 0.02) fp16 weights",
        "impl": "reference",
        "config": bench_config(a.batch, layers, f"inputs larger than L2: {r['weight_bytes'] / 1e9:.2f} GB of weights read per step",
                               kv_dtype="fp16", page_size=None),
        "clocks": clocks.summary(),
        "e2e": {"value": round(a.batch / r["e2e_ms_per_step"] * 1e3, 1), "unit": "tok/s",
                "ms_per_step": round(r["e2e_ms_per_step"], 4), "h2d_bytes_per_step": 0, "d2h_bytes_per_step": a.batch * 4},
        "prefill": {"value": round(PREFILL_TOKENS / pre_ms * 1e3, 1), "tokens": PREFILL_TOKENS, "ms": round(pre_ms, 4),
                    "frac": round(prefill_flops(layers) / (pre_ms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4),
                    "peak_tflops": pk["bf16_tflops"], "peaks": pk["source"]},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4), "peaks": pk["source"],
                     "bytes_per_step": int(step_bytes), "mean_context": mean_ctx},
        "points": {k: round(v, 1) for k, v in r["points"].items()},
    }
    print(json.dumps(out))
    return 0


def bench_config(batch: int, layers: int, l2: str, kv_dtype: str = "bf16", page_size=PAGE) -> dict:
    return {"model": SHAPE_NAME, "layers": layers, "layers_full": MODEL["num_hidden_layers"],
            "hidden": MODEL["hidden_size"], "heads": MODEL["num_attention_heads"],
            "kv_heads": MODEL["num_key_value_heads"], "head_dim": MODEL["head_dim"],
            "intermediate": MODEL["intermediate_size"], "vocab": MODEL["vocab_size"], "global_batch": batch,
            "seq_len": CONTEXT_LEN, "prompt_len": PROMPT_LEN, "page_size": page_size, "kv_dtype": kv_dtype,
            "parallelism": "single GPU", "l2": l2}


def main() -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawTextHelpFormatter)
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--layers", type=int, default=None,
                    help="fewer layers than the configuration has (both numbers are reported)")
    ap.add_argument("--shape", default="1b", choices=sorted(SHAPES), help="layer sizes: 1b (the default run), 3b, 8b")
    ap.add_argument("--prompt", type=int, default=PROMPT_LEN, help="tokens of each prompt behind the decode steps")
    ap.add_argument("--prefill-tokens", type=int, default=PREFILL_TOKENS, help="tokens of the timed prefill step")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="decode", choices=["decode", "mixed"],
                    help="decode: the default run; mixed: requests of random lengths through the scheduler (see mixed_workload)")
    ap.add_argument("--requests", type=int, default=32, help="mixed: number of requests")
    ap.add_argument("--new", type=int, default=128, help="mixed: tokens generated per request")
    ap.add_argument("--max-prefill", type=int, default=512, help="mixed: token budget of a step")
    ap.add_argument("--pool-fraction", type=float, default=1.0, help="mixed: fraction of the pages all requests would need (< 1: preemptions)")
    ap.add_argument("--no-points", action="store_true", help="skip the batch-1 and batch-64 decode points")
    ap.add_argument("--breakdown", action="store_true", help="print per-kernel times of a decode step and exit")
    ap.add_argument("--prefill", action="store_true", help="with --breakdown: the prefill step instead of a decode step")
    a = ap.parse_args()
    if a.impl == "reference":
        return reference_arm(a)
    if a.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {a.gpus} is not supported")
        return 2
    if a.warmup < 3:
        a.warmup = 3
    if (a.shape, a.prompt, a.prefill_tokens) != ("1b", PROMPT_LEN, PREFILL_TOKENS):
        choose_shape(a.shape, a.prompt, a.prefill_tokens, a.steps + a.warmup + 8)
    if a.layers is None:
        a.layers = MODEL["num_hidden_layers"]
    if a.breakdown:
        return breakdown(a.layers, a.batch, a.prefill)
    if a.workload == "mixed":
        return mixed_workload(a)
    import torch

    pk = peaks()
    point_batches = [] if a.no_points else [b for b in (1, 64) if b != a.batch]
    max_batch = max([a.batch] + point_batches)
    eng = build_engine(a.layers, max_batch, a.steps + a.warmup + 8)
    clocks = ClockSampler().start()
    ms, mean_ctx, launches = decode_device(eng, a.batch, a.steps, a.warmup, clocks)
    value = a.batch / ms * 1e3
    step_bytes = eng.weight_bytes + a.batch * mean_ctx * eng.kv_bytes_per_token
    achieved = step_bytes / ms / 1e6
    points = {f"decode_b{a.batch}": round(value, 1)}
    for b in point_batches:      # the median of three short runs
        pms = statistics.median(decode_device(eng, b, min(a.steps, 64), a.warmup)[0] for _ in range(3))
        points[f"decode_b{b}"] = round(b / pms * 1e3, 1)
    pre_ms = prefill_device(eng, 3, 5)
    pre_frac = prefill_flops(a.layers) / (pre_ms * 1e-3) / (pk["bf16_tflops"] * 1e12)
    e2e_ms, h2d, d2h = decode_e2e(eng, a.batch, min(a.steps, 64), a.warmup)
    finite, drift, cosine = self_check(eng)
    # A guard against a timed path that computes something else, not a test of rounding: two bfloat16 paths drift apart
    # with depth (1.5e-2 of the largest logit at 16 layers of the 1B shape, 3.3e-2 at the 32 layers of the 8B shape,
    # where the 32-bit path of the same engine lies 4.9e-2 from both), so the drift is reported and the cosine judged.
    if not finite or cosine < 0.995:
        print(f"bench.py: the timed path's logits are wrong (finite: {finite}; decode steps against a whole prompt: "
              f"cosine {cosine:.5f}, {drift:.3e} of the largest logit apart)", file=sys.stderr)
        return 1
    out = {
        "metric": f"decode tok/s at batch {a.batch} ({SHAPE_NAME}, {PROMPT_LEN:,}-token prompts)",
        "value": round(value, 1), "unit": "tok/s", "n_gpus": 1, "steps": a.steps, "warmup": a.warmup,
        "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: uniform-random token ids, random N(0, 0.02) bf16 weights",
        "impl": "ours",
        "config": bench_config(a.batch, a.layers, f"inputs larger than L2: {eng.weight_bytes / 1e9:.2f} GB of weights read per step"),
        "clocks": clocks.summary(),
        "e2e": {"value": round(a.batch / e2e_ms * 1e3, 1), "unit": "tok/s", "ms_per_step": round(e2e_ms, 4),
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
        "gpu_launches": int(round(launches * a.steps)),
        "prefill": {"value": round(PREFILL_TOKENS / pre_ms * 1e3, 1), "tokens": PREFILL_TOKENS, "ms": round(pre_ms, 4),
                    "frac": round(pre_frac, 4), "peak_tflops": pk["bf16_tflops"], "peaks": pk["source"]},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4), "peaks": pk["source"],
                     "bytes_per_step": int(step_bytes), "mean_context": mean_ctx},
        "points": points,
        "check": {"finite": finite, "decode_vs_whole": round(drift, 6), "cosine": round(cosine, 6)},
    }
    eng.close()
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
