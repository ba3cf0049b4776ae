"""Trace replay: feeds given token ids through the model step by step and writes logits. It
samples nothing and has no forward pass, cache or loader of its own: it drives `ModelRunner`,
the step function that generation uses.

Steps come on standard input, one JSON object a line:

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

All entries of a step are one batch. For a step in which something is wanted the logits at
the wanted places (in the order of the entries and of `want`) go to `<out>/<step>.f32` as
little-endian float32 [wanted, vocab]. After every step a line `done <step>` is printed and
flushed. `end` names requests that are finished after the step; their pages are given back.
With --planes every step also leaves its layers' named planes (parts/planes.py) beside the logits, so
that the first (layer, sub-step) at which two runs part ways can be read off; the reference's
scripts/layer_diff.py does that for its own graph.

The reference's nearest things: `RefEngine.forward` keeps its cache between calls
(scripts/ref_engine.py:218-232) and `hi_prefill(slot, tokens, T, p0)` continues a slot at p0
(src/api.cu:1767-1771).
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import numpy as np


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    ap.add_argument("--out", required=True, help="folder for <step>.f32 files")
    ap.add_argument("--max-tokens", type=int, required=True,
                    help="most tokens live requests hold at any time (each rounded up to 64); sizes the cache pool")
    ap.add_argument("--page-size", type=int, default=16)
    ap.add_argument("--max-requests", type=int, default=4, help="most requests live at a time")
    ap.add_argument("--planes", action="store_true",
                    help="also write <step>.planes.safetensors: every layer's named planes of the step's rows "
                         "(parts/planes.py), named <order index>.<plane>; such steps run eagerly")
    a = ap.parse_args(argv)

    from .runner import ModelRunner
    from .batch import StepEntry
    from ..kernels import library, ops
    import torch

    os.makedirs(a.out, exist_ok=True)
    library.load("core")
    if 64 % a.page_size:
        raise SystemExit("trace_run: --page-size must divide 64")
    num_pages = -(-a.max_tokens // 64) * (64 // a.page_size)
    runner = ModelRunner.from_folder(a.model, dtype=a.dtype, page_size=a.page_size, num_pages=num_pages,
                                     max_num_seqs=a.max_requests)
    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        rec = json.loads(line)
        step = rec["step"]
        entries = [StepEntry(e["id"], e["tokens"], e.get("want", [])) for e in rec.get("entries", [])]
        dump = {} if a.planes else None
        logits = runner.step(entries, dump=dump)
        if dump:
            from safetensors.torch import save_file

            save_file({f"{i}.{name}": t.cpu().contiguous() for (i, name), t in dump.items()},
                      os.path.join(a.out, f"{step}.planes.safetensors"))
        if logits.shape[0]:
            arr = logits.detach().to("cpu").numpy().astype("<f4", copy=False)
            arr.tofile(os.path.join(a.out, f"{step}.f32"))
        else:
            torch.cuda.synchronize()
        ops.check_device_status()              # a kernel that gave up on a bounded wait ends the replay with an error
        for rid in rec.get("end", []):
            runner.end(rid)
        print(f"done {step}", flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
