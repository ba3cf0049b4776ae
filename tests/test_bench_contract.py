"""The parts of bench.py's contract that need no GPU: more than one GPU is refused with one line
and exit code 2, the reference arm prints an `unavailable` line and exits 0 where it cannot run
(no GPU), the weight file it writes for the reference has the reference's layout, and the other
layer shapes are whole configurations of the architecture. With a GPU: the reference arm prints
the same kind of line as the engine's own arm."""
import json
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def run_bench(*args):
    return subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), *args], capture_output=True, text=True, timeout=120)


def test_more_than_one_gpu_is_refused():
    r = run_bench("--gpus", "2")
    assert r.returncode == 2
    assert len(r.stdout.strip().splitlines()) == 1 and "one GPU" in r.stdout


def test_reference_arm_without_a_gpu_says_so():
    import torch

    if torch.cuda.is_available():
        pytest.skip("a GPU is visible: the reference arm runs (see the gpu test below)")
    r = run_bench("--impl", "reference", "--gpus", "1", "--steps", "2", "--warmup", "1")
    assert r.returncode == 0
    line = json.loads(r.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and "CUDA" in line["unavailable"] and "\n" not in line["unavailable"]


def test_reference_weight_file_layout(tmp_path):
    """The random flat file for the reference: header fields as scripts/export.py:230-232 packs them, every
    tensor padded to 256 bytes (export.py:251-253), the size the layout implies; the untied file has a head."""
    import struct

    sys.path.insert(0, os.path.join(ROOT, "baseline"))
    import reference_arm as ra

    m = dict(vocab_size=96, hidden_size=64, intermediate_size=48, num_attention_heads=4, num_key_value_heads=2,
             head_dim=16, max_position_embeddings=128, rms_norm_eps=1e-5, rope_theta=10000.0, rope_scaling=None,
             tie_word_embeddings=True)
    pad = lambda n: -(-n // 256) * 256
    sizes = {}
    for tied in (True, False):
        path = str(tmp_path / f"w{int(tied)}.bin")
        sizes[tied] = ra.write_random_weights(path, dict(m, tie_word_embeddings=tied), layers=3)
        raw = open(path, "rb").read(64)
        h = struct.unpack("<10i2f2i", raw[:56])
        assert h[:10] == (0x48495046, 2, 96, 64, 48, 3, 4, 2, 16, 128) and h[12] == int(tied) and h[13] == 0
        assert abs(h[10] - 1e-5) < 1e-12 and h[11] == 1.0
    layer = 2 * pad(64 * 2) + pad(8 * 16 * 64 * 2) + pad(64 * 64 * 2) + pad(96 * 64 * 2) + pad(64 * 48 * 2)
    want = 64 + pad(8 * 4) + pad(96 * 64 * 2) + pad(64 * 2) + 3 * layer
    assert sizes[True] == want and sizes[False] == want + pad(96 * 64 * 2)
    inv = ra.llama3_inv_freq(16, 10000.0, None)
    assert inv[0] == 1.0 and abs(inv[1] - 10000.0 ** (-2 / 16)) < 1e-15


@pytest.mark.gpu
def test_reference_arm_prints_the_bench_line():
    """Two layers of the 1B shape through the reference's own library: a value, or one line that says why not."""
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--layers", "2", "--steps", "4",
                        "--warmup", "3", "--no-points"], capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stderr[-2000:]
    line = json.loads(r.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference"
    if "unavailable" in line:
        assert isinstance(line["unavailable"], str) and "\n" not in line["unavailable"]
        return
    assert line["value"] > 0 and line["prefill"]["ms"] > 0 and line["e2e"]["value"] > 0
    assert line["config"]["layers"] == 2 and line["config"]["layers_full"] == 16


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
