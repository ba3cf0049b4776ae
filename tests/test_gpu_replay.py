"""Trace replay through bin/trace_run, in 32-bit and in bfloat16, on two tiny configurations:
the same requests whole, with the last 32 tokens decoded one by one, in portions of changing
size, and mixed with other requests on so few pages that they are used again. Every position's
logits are compared with the plain implementation."""
import pytest
import torch

import plain_llama as plain
import tiny

pytestmark = pytest.mark.gpu

LENGTHS = {"a": [5, 11, 17, 64, 100, 128, 33, 90], "b": [1, 7, 33, 64, 200, 256, 150, 81],
           "c": [700, 130, 64, 257, 400, 16, 33, 90]}


@pytest.fixture(scope="module", params=[("a", "float32"), ("b", "float32"), ("c", "float32"), ("a", "bfloat16"), ("b", "bfloat16"),
                                        ("c", "bfloat16")],
                ids=lambda p: f"{p[0]}-{p[1]}")
def setup(request, tmp_path_factory):
    which, dtype = request.param
    folder = tiny.make_model_folder(tmp_path_factory.mktemp(f"model_{which}_{dtype}"), which,
                                    torch.float32 if dtype == "float32" else torch.bfloat16)
    cfg, weights = plain.read_model(folder)
    vocab = cfg["vocab_size"]
    requests = {f"r{i}": tiny.random_tokens(n, vocab, 100 + i) for i, n in enumerate(LENGTHS[which])}
    ref = {rid: plain.forward(cfg, weights, toks) for rid, toks in requests.items()}
    # room for four live requests of the longest kind, rounded up to 64 each: pages are used again
    longest = -(-max(LENGTHS[which]) // 64) * 64
    tr = tiny.TraceRun(folder, dtype, tmp_path_factory.mktemp(f"out_{which}_{dtype}"), 4 * longest)
    yield dict(which=which, dtype=dtype, requests=requests, ref=ref, tr=tr)
    tr.close()


def _check(setup, plan, what):
    got = tiny.run_plan(setup["tr"], setup["requests"], plan)
    for rid, ref in setup["ref"].items():
        tiny.assert_logits_close(got[rid], ref, setup["dtype"], f"{what} {setup['which']} {setup['dtype']} {rid}",
                                 group=(f"tiny {setup['which']}", what))


def test_whole(setup):
    _check(setup, tiny.plan_whole(setup["requests"]), "whole")


def test_tail_one_by_one(setup):
    _check(setup, tiny.plan_tail_decode(setup["requests"], 32), "tail")


def test_portions(setup):
    _check(setup, tiny.plan_portions(setup["requests"]), "portions")


@pytest.mark.parametrize("seed", [0, 1, 2])
def test_mixed(setup, seed):
    _check(setup, tiny.plan_mixed(setup["requests"], seed), f"mixed{seed}")


@pytest.mark.parametrize("seed", [0, 1, 2])
def test_mixed_long_portions(setup, seed):
    """The scheduler's ordinary step: a portion of more than 64 rows of one request (where it has that many left)
    beside short portions and single decode rows of the others, on a pool so small that pages are used again."""
    plan = tiny.plan_mixed_long(setup["requests"], seed)
    if setup["which"] == "c":
        mixed = [s for s in plan if any(n > 64 for _, n in s) and any(n == 1 for _, n in s)]
        assert mixed, "the plan has no step with a long portion beside a decode row"
    _check(setup, plan, f"mixed-long{seed}")


def test_wanted_subset_and_no_want(setup):
    """`want` may be empty or name a few places; nothing is written for a step that wants nothing."""
    tr, (rid, toks) = setup["tr"], list(setup["requests"].items())[3]
    ref = setup["ref"][rid]
    n = len(toks)
    assert tr.step([("w", toks[:10], [])]) is None
    got = tr.step([("w", toks[10:n], [0, n - 11])], end=["w"])
    tiny.assert_logits_close(got, ref[[10, n - 1]], setup["dtype"], "subset")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("which", ["d", "e"])
def test_sizes_the_fast_kernels_take_only_in_part(which, dtype, tmp_path):
    """Heads of 48 and of 80, a group of 7, widths that are no multiple of 32 or 64, odd vocabularies: whatever a
    tensor-core kernel does not take goes to another kernel, never to a wrong result. Whole, in portions, with the
    last tokens one by one, and mixed on a small pool, through the step function in this process."""
    from hipinfer_b200.engine import ModelRunner

    folder = tiny.make_model_folder(tmp_path / "m", which, torch.float32 if dtype == "float32" else torch.bfloat16)
    cfg, weights = plain.read_model(folder)
    requests = {f"o{i}": tiny.random_tokens(n, cfg["vocab_size"], 300 + i) for i, n in enumerate([130, 9, 64, 33, 200, 17])}
    ref = {rid: plain.forward(cfg, weights, toks) for rid, toks in requests.items()}
    runner = ModelRunner.from_folder(folder, dtype=dtype, page_size=16, num_pages=4 * 208 // 16, max_model_len=256, max_num_seqs=4)
    st = tiny.RunnerStepper(runner)
    for name, plan in (("whole", tiny.plan_whole(requests)), ("portions", tiny.plan_portions(requests)),
                       ("tail", tiny.plan_tail_decode(requests, 32)), ("mixed", tiny.plan_mixed(requests, 1)),
                       ("mixed-long", tiny.plan_mixed_long(requests, 2))):
        got = tiny.run_plan(st, requests, plan)
        for rid in requests:
            tiny.assert_logits_close(got[rid], ref[rid], dtype, f"{which} {name} {rid}", group=(f"tiny {which}", name))
        runner.cache.check()
        assert runner.cache.free_pages() == [52]
