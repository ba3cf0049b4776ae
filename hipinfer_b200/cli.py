"""Command line. The reference's only generating `main` is its oracle's
(scripts/ref_engine.py:248-257: --weights, --tokens, --new, --mode); the same option names
are kept, with --model for a folder of config.json and model.safetensors.

    python -m hipinfer_b200 generate --model DIR --tokens 1 2 3 --new 8 [--mode bf16|fp32]
                                     [--temperature T --seed S] [--max-batch --max-seq --max-prefill]
    python -m hipinfer_b200 random-model --config config.json --out DIR --seed 0 [--std 0.02] [--dtype bfloat16]
    python -m hipinfer_b200 replay --model DIR --dtype bfloat16 --out DIR --max-tokens N   (steps on stdin)
    python -m hipinfer_b200 bench [bench.py's options]        (the measurement program beside the package)
"""
from __future__ import annotations

import argparse
import json
import sys


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="hipinfer_b200", description=__doc__, formatter_class=argparse.RawTextHelpFormatter)
    sub = ap.add_subparsers(dest="cmd", required=True)
    g = sub.add_parser("generate", help="generate tokens after a prompt of token ids")
    g.add_argument("--model", "--weights", dest="model", required=True)
    g.add_argument("--tokens", type=int, nargs="+", default=[1, 2, 3, 4])
    g.add_argument("--new", type=int, default=8)
    g.add_argument("--mode", "--dtype", dest="mode", default="bf16", choices=["bf16", "fp32", "bfloat16", "float32"])
    g.add_argument("--temperature", type=float, default=0.0)
    g.add_argument("--seed", type=int, default=0)
    g.add_argument("--max-batch", type=int, default=8)
    g.add_argument("--max-seq", type=int, default=2048)
    g.add_argument("--max-prefill", type=int, default=1024)
    r = sub.add_parser("random-model", help="write a model folder with seeded random weights")
    r.add_argument("--config", required=True, help="a config.json of a registered architecture")
    r.add_argument("--out", required=True)
    r.add_argument("--seed", type=int, default=0)
    r.add_argument("--std", type=float, default=0.02)
    r.add_argument("--norm-std", type=float, default=0.0)
    r.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    sub.add_parser("replay", help="trace replay; same options as bin/trace_run", add_help=False)
    sub.add_parser("bench", help="the measurement program (bench.py beside the package); same options", add_help=False)
    if argv is None:
        argv = sys.argv[1:]
    if argv and argv[0] == "replay":
        from .engine.replay import main as replay_main

        return replay_main(argv[1:])
    if argv and argv[0] == "bench":
        import os
        import runpy

        script = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "bench.py")
        if not os.path.isfile(script):
            print(f"hipinfer_b200 bench: {script} is not there (the measurement program lives beside the package)", file=sys.stderr)
            return 2
        sys.argv = [script] + list(argv[1:])
        try:
            runpy.run_path(script, run_name="__main__")
        except SystemExit as e:
            return int(e.code or 0)
        return 0
    a = ap.parse_args(argv)
    if a.cmd == "generate":
        from .engine.api import Engine

        eng = Engine(a.model, max_batch=a.max_batch, max_seq=a.max_seq, max_prefill=a.max_prefill, dtype=a.mode)
        print({k: getattr(eng, k) for k in ("vocab", "hidden", "inter", "layers", "heads", "kv_heads", "head_dim",
                                            "max_pos", "tied")})
        print(eng.generate(a.tokens, a.new, temperature=a.temperature, seed=a.seed))
        eng.close()
        return 0
    if a.cmd == "random-model":
        import torch

        from .config import config_from_dict
        from .weights import write_random_model

        with open(a.config) as f:
            cfg = config_from_dict(json.load(f))
        write_random_model(cfg, a.out, a.seed, a.std, a.norm_std, getattr(torch, a.dtype))
        print(a.out)
        return 0
    return 2


if __name__ == "__main__":
    sys.exit(main())
