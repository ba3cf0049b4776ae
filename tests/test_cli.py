"""The command line as a user runs it: child processes of `python -m hipinfer_b200` and `bin/hipinfer-b200`.
random-model writes the folder the library call writes; generate prints the tokens of the plain implementation
(the reference's oracle has the same options: scripts/ref_engine.py:248-257); bench refuses more than one GPU."""
import ast
import json
import os
import subprocess
import sys

import pytest
import torch

import plain_llama as plain
import tiny

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def run(args, timeout=600):
    env = dict(os.environ, PYTHONPATH=ROOT + os.pathsep + os.environ.get("PYTHONPATH", ""))
    return subprocess.run(args, capture_output=True, text=True, timeout=timeout, env=env, cwd=ROOT)


def make_folder(tmp_path, which, via_module=True):
    w = tiny.WEIGHTS[which]
    cfg_path = tmp_path / "cfg.json"
    cfg_path.write_text(json.dumps(w["cfg"]))
    out = tmp_path / "model"
    head = [sys.executable, "-m", "hipinfer_b200"] if via_module else [sys.executable, os.path.join(ROOT, "bin", "hipinfer-b200")]
    r = run(head + ["random-model", "--config", str(cfg_path), "--out", str(out), "--seed", str(w["seed"]), "--std",
                    str(w["std"]), "--norm-std", str(w["norm_std"])])
    assert r.returncode == 0, r.stderr[-2000:]
    assert r.stdout.strip().splitlines()[-1] == str(out)
    return str(out)


def test_random_model_writes_what_the_library_writes(tmp_path):
    from hipinfer_b200.weights import ModelFiles

    folder = make_folder(tmp_path, "b")
    same = tiny.make_model_folder(tmp_path / "lib", "b", torch.bfloat16)
    assert json.load(open(os.path.join(folder, "config.json"))) == json.load(open(os.path.join(same, "config.json")))
    a, b = ModelFiles(folder), ModelFiles(same)
    assert sorted(a.names()) == sorted(b.names())
    for n in a.names():
        assert torch.equal(a.get(n), b.get(n)), n
    a.close()
    b.close()


def test_bad_arguments_end_with_a_message(tmp_path):
    r = run([sys.executable, "-m", "hipinfer_b200", "random-model", "--config", str(tmp_path / "none.json"), "--out", str(tmp_path)])
    assert r.returncode != 0 and "none.json" in r.stderr
    r = run([sys.executable, "-m", "hipinfer_b200", "bench", "--gpus", "2"])
    assert r.returncode == 2 and "one GPU" in r.stdout


@pytest.mark.gpu
@pytest.mark.parametrize("which,mode,via_module", [("a", "fp32", True), ("b", "bf16", False)])
def test_generate_prints_the_plain_tokens(tmp_path, which, mode, via_module):
    folder = make_folder(tmp_path, which, via_module)
    cfg, weights = plain.read_model(folder)
    prompt = tiny.random_tokens(19, cfg["vocab_size"], 5)
    want, steps = plain.generate_greedy(cfg, weights, prompt, 6)
    head = [sys.executable, "-m", "hipinfer_b200"] if via_module else [sys.executable, os.path.join(ROOT, "bin", "hipinfer-b200")]
    r = run(head + ["generate", "--model", folder, "--tokens", *map(str, prompt), "--new", "6", "--mode", mode,
                    "--max-seq", "64", "--max-batch", "2", "--max-prefill", "8"])
    assert r.returncode == 0, r.stderr[-2000:]
    lines = r.stdout.strip().splitlines()
    shape = ast.literal_eval(lines[-2])
    assert shape["vocab"] == cfg["vocab_size"] and shape["layers"] == cfg["num_hidden_layers"]
    got = ast.literal_eval(lines[-1])
    if mode == "fp32":
        assert got == want
    else:       # bfloat16: the same token unless the plain implementation's two best logits nearly tie there
        for i, (g, w) in enumerate(zip(got, want)):
            if g != w:
                top = torch.topk(steps[i].float(), 2).values
                assert float(top[0] - top[1]) < 0.02 * float(steps[i].abs().max()), (i, got, want)
                break
        assert len(got) == len(want)
