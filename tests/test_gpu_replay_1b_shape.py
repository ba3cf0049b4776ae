"""Replay at the real layer sizes of the Llama-3.2-1B shape: width 2,048, 32 query and 8 key/value heads of 64,
feed-forward 8,192, vocabulary 128,256, llama3 frequency scaling (factor 32, original 8,192), tied head,
with 2 of its 16 layers (tiny.LLAMA_1B_LAYERS_TESTED of tiny.LLAMA_1B_LAYERS_FULL) so that the plain
implementation on the CPU stays within seconds. At these sizes the engine takes the kernels and plans that
the tiny configurations never reach: the 8- and 16-slice products of decode steps, the CTA-pair product and
the rotation in the q/k/v product's epilogue for long portions, the two-stage sampler, the 128,256-wide
head. The same requests whole, with the last 32 tokens one by one, in portions down to two tokens, and
mixed (short portions; and long portions beside decode rows) on a pool of four times the longest request,
in 32-bit and in bfloat16, every position compared with the plain implementation. One request also goes
through bin/trace_run. The reference runs its end-to-end gate on the real model too (tests/gate.py:170-189)."""
import pytest
import torch

import plain_llama as plain
import tiny

pytestmark = pytest.mark.gpu

LENGTHS = [384, 130, 70, 257, 33, 200]


@pytest.fixture(scope="module")
def model(tmp_path_factory):
    folder = tiny.make_model_folder(tmp_path_factory.mktemp("model_1b2l"), "1b2l", torch.bfloat16)
    cfg, weights = plain.read_model(folder)
    assert cfg["num_hidden_layers"] == tiny.LLAMA_1B_LAYERS_TESTED < tiny.LLAMA_1B_LAYERS_FULL
    requests = {f"r{i}": tiny.random_tokens(n, cfg["vocab_size"], 300 + i) for i, n in enumerate(LENGTHS)}
    ref = {rid: plain.forward(cfg, weights, toks) for rid, toks in requests.items()}
    return dict(folder=folder, cfg=cfg, requests=requests, ref=ref)


@pytest.fixture(scope="module", params=["float32", "bfloat16"])
def setup(request, model):
    from hipinfer_b200.engine import ModelRunner

    dtype = request.param
    longest = -(-max(LENGTHS) // 64) * 64
    runner = ModelRunner.from_folder(model["folder"], dtype=dtype, page_size=16, num_pages=4 * longest // 16,
                                     max_num_seqs=4, max_model_len=1024)
    yield dict(model, dtype=dtype, stepper=tiny.RunnerStepper(runner))
    del runner
    torch.cuda.empty_cache()


def _check(setup, plan, what):
    from hipinfer_b200.kernels import ops

    got = tiny.run_plan(setup["stepper"], setup["requests"], plan)
    ops.check_device_status()
    for rid, ref in setup["ref"].items():
        tiny.assert_logits_close(got[rid], ref, setup["dtype"], f"1b-shape-2-layers {what} {rid}",
                                 group=("1B shape, 2 layers", what))


def test_whole(setup):
    _check(setup, tiny.plan_whole(setup["requests"]), "whole")


def test_tail_one_by_one(setup):
    _check(setup, tiny.plan_tail_decode(setup["requests"], 32), "tail")


def test_portions(setup):
    _check(setup, tiny.plan_portions(setup["requests"]), "portions")


def test_mixed(setup):
    _check(setup, tiny.plan_mixed(setup["requests"], 0), "mixed")


def test_mixed_long_portions(setup):
    plan = tiny.plan_mixed_long(setup["requests"], 0)
    assert [s for s in plan if any(n > 64 for _, n in s) and any(n == 1 for _, n in s)]
    _check(setup, plan, "mixed-long")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_through_trace_run(model, dtype, tmp_path):
    """The replay program itself at these sizes: one request, most of it in one step, then token by token."""
    rid, toks = "r2", model["requests"]["r2"]
    tr = tiny.TraceRun(model["folder"], dtype, tmp_path, 128)
    n = len(toks)
    got = [tr.step([(rid, toks[:n - 3], [n - 5, n - 4])])]
    for i in range(n - 3, n):
        got.append(tr.step([(rid, toks[i:i + 1], [0])], end=[rid] if i == n - 1 else []))
    tr.close()
    tiny.assert_logits_close(torch.cat(got), model["ref"][rid][[n - 5, n - 4, n - 3, n - 2, n - 1]], dtype,
                             f"1b-shape-2-layers trace_run {rid}", group=("1B shape, 2 layers", "trace_run"))
