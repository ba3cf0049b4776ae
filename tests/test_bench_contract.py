"""The parts of bench.py's contract that need no GPU: more than one GPU is refused with one line
and exit code 2, the reference arm prints its `unavailable` line and exits 0, and the other layer
shapes are whole configurations of the architecture."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def run_bench(*args):
    return subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), *args], capture_output=True, text=True, timeout=120)


def test_more_than_one_gpu_is_refused():
    r = run_bench("--gpus", "2")
    assert r.returncode == 2
    assert len(r.stdout.strip().splitlines()) == 1 and "one GPU" in r.stdout


def test_reference_arm_says_why_it_is_unavailable():
    r = run_bench("--impl", "reference", "--gpus", "1", "--steps", "2", "--warmup", "1")
    assert r.returncode == 0
    line = json.loads(r.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and isinstance(line["unavailable"], str) and "\n" not in line["unavailable"]


def test_other_shapes_are_whole_configurations():
    sys.path.insert(0, ROOT)
    import importlib

    import bench
    from hipinfer_b200.config import config_from_dict

    try:
        for shape, heads, head_dim in (("3b", 24, 128), ("8b", 32, 128)):
            importlib.reload(bench)
            bench.choose_shape(shape, 4096, 8192, 100)
            cfg = config_from_dict(dict(bench.MODEL))
            assert (cfg.num_attention_heads, cfg.head_dim) == (heads, head_dim)
            assert bench.CONTEXT_LEN >= 8192 + 100 and bench.PROMPT_LEN == 4096 and bench.PREFILL_TOKENS == 8192
            assert bench.SHAPE_NAME != "Llama-3.2-1B shape"
        assert bench.MODEL["rope_scaling"]["factor"] == 8.0 and not bench.MODEL["tie_word_embeddings"]
    finally:
        importlib.reload(bench)
