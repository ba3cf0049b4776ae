"""The engine through its own entry points, in 32-bit and in bfloat16: greedy and temperature
generation against the plain implementation, batches, the scheduler on so few pages that it has
to preempt, long decoding across pages and key chunks, the first tokens of a sequence, and the
reference-style slot calls."""
import pytest
import torch

import plain_llama as plain
import tiny

pytestmark = pytest.mark.gpu
DTYPES = ["float32", "bfloat16"]


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    out = {}
    for which in ("a", "b", "c"):
        f = tiny.make_model_folder(tmp_path_factory.mktemp(f"eng_{which}"), which, torch.bfloat16)
        out[which] = (f,) + plain.read_model(f)
    return out


def engine(folder, dtype, **kw):
    from hipinfer_b200 import Engine

    return Engine(folder, dtype=dtype, **kw)


def check_tokens(got, want, steps, dtype, what):
    """Token identity; in bfloat16 a different token is accepted only where the plain
    implementation's two best logits nearly tie (the reference's gate does the same against its
    own oracle, tests/gate.py:68-89), and nothing after the first such place is compared."""
    for i, (g, w) in enumerate(zip(got, want)):
        if g == w:
            continue
        top = torch.topk(steps[i].float(), 2).values
        gap = float(top[0] - top[1]) / float(steps[i].abs().max())
        assert dtype == "bfloat16" and gap < 0.02, f"{what}: token {i} is {g}, plain {w} (relative gap {gap:.4f})"
        return
    assert len(got) == len(want)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("which,n_prompt,n_new", [("a", 5, 8), ("a", 17, 8), ("b", 33, 12), ("c", 70, 10)])
def test_greedy_generation(folders, which, n_prompt, n_new, dtype):
    folder, cfg, w = folders[which]
    prompt = tiny.random_tokens(n_prompt, cfg["vocab_size"], 7 + n_prompt)
    want, steps = plain.generate_greedy(cfg, w, prompt, n_new)
    eng = engine(folder, dtype, max_batch=2, max_seq=128, max_prefill=16)   # the prompt is cut into portions of 16
    got = eng.generate(prompt, n_new)
    eng.close()
    check_tokens(got, want, steps, dtype, f"{which} {dtype}")


@pytest.mark.parametrize("dtype", DTYPES)
def test_batch_of_prompts_and_temperature(folders, dtype):
    """Tiny B's workload: prompts of 1/7/33/64 tokens in portions of 16 beside decode tokens,
    12 steps at temperature 0.8, seed 4. Every drawn token must be the arg max of the plain
    implementation's noisy scores at that position (within rounding of the logits)."""
    folder, cfg, w = folders["b"]
    prompts = [tiny.random_tokens(n, cfg["vocab_size"], 3 + i) for i, n in enumerate((1, 7, 33, 64))]
    eng = engine(folder, dtype, max_batch=4, max_seq=256, max_prefill=16)
    outs = eng.generate(prompts, 12, temperature=0.8, seed=4)
    eng.close()
    tol = 1e-3 if dtype == "float32" else 0.08
    for p, out in zip(prompts, outs):
        assert len(out) == 12
        seq = list(p)
        for tok in out:
            logits = plain.forward(cfg, w, seq)[-1]
            sc = plain.gumbel_scores(logits, 0.8, 4, len(seq))
            assert float(sc.max() - sc[tok]) <= tol * float(logits.abs().max()) / 0.8, f"token {tok} at position {len(seq)}"
            seq.append(tok)
    # the same prompts one at a time draw the same tokens: a draw does not depend on the batch
    if dtype == "float32":
        eng = engine(folder, dtype, max_batch=1, max_seq=256, max_prefill=64)
        assert [eng.generate(p, 12, temperature=0.8, seed=4) for p in prompts] == outs
        eng.close()


@pytest.mark.parametrize("dtype", DTYPES)
def test_scheduler_preempts_when_pages_run_out(folders, dtype):
    """Four requests on a pool that cannot hold them all to the end: the youngest is preempted
    and computed again, and everyone still produces the tokens of an engine with room to spare."""
    folder, cfg, w = folders["a"]
    prompts = [tiny.random_tokens(n, cfg["vocab_size"], 40 + i) for i, n in enumerate((30, 25, 28, 20))]
    roomy = engine(folder, dtype, max_batch=4, max_seq=128, max_prefill=32)
    want = roomy.generate(prompts, 40)
    roomy.close()
    tight = engine(folder, dtype, max_batch=4, max_seq=128, max_prefill=32, num_pages=13)  # 208 tokens for 4 x ~67
    got = tight.generate(prompts, 40)
    assert tight.scheduler.n_preemptions > 0
    tight.runner.cache.check()
    assert tight.runner.cache.free_pages() == [13] and tight.runner.cache.slots.free_count == 4
    tight.close()
    if dtype == "float32":
        assert got == want
    else:
        for g, wnt, p in zip(got, want, prompts):
            if g != wnt:        # recomputation goes through the prefill kernels: only a near-tie may differ
                i = next(j for j in range(40) if g[j] != wnt[j])
                logits = plain.forward(cfg, w, p + wnt[:i])[-1]
                top = torch.topk(logits, 2).values
                assert float(top[0] - top[1]) < 0.02 * float(logits.abs().max())


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding_across_pages_and_chunks(folders, dtype):
    """A 150-token prompt, then 450 tokens one by one: the logits of every decoded position against
    the plain implementation on the whole sequence (positions cross many pages and the 256-key
    chunks of the row-attention kernels)."""
    from hipinfer_b200.engine import ModelRunner, StepEntry

    folder, cfg, w = folders["c"]
    toks = tiny.random_tokens(600, cfg["vocab_size"], 77)
    ref = plain.forward(cfg, w, toks)
    runner = ModelRunner.from_folder(folder, dtype=dtype, max_model_len=1024, max_num_seqs=2)
    got = [runner.step([StepEntry("r", toks[:150], [149])]).float().cpu()]
    for i in range(150, 600):
        got.append(runner.step([StepEntry("r", [toks[i]], [0])]).float().cpu())
    got = torch.cat(got)
    tiny.assert_logits_close(got, ref[149:], dtype, f"long decode {dtype}")
    runner.end("r")
    runner.cache.check()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("which", ["a", "b", "c"])
def test_first_tokens_of_a_sequence(folders, which, dtype):
    from hipinfer_b200.engine import ModelRunner, StepEntry

    folder, cfg, w = folders[which]
    toks = tiny.random_tokens(4, cfg["vocab_size"], 5)
    ref = plain.forward(cfg, w, toks)
    runner = ModelRunner.from_folder(folder, dtype=dtype, max_model_len=64, max_num_seqs=4)
    one = runner.step([StepEntry("one", toks[:1], [0])]).float().cpu()
    tiny.assert_logits_close(one, ref[:1], dtype, "a request of one token")
    whole = runner.step([StepEntry("w", toks, [0, 1, 2, 3])]).float().cpu()
    tiny.assert_logits_close(whole, ref, dtype, "four tokens at once")
    step = torch.cat([runner.step([StepEntry("s", [t], [0])]).float().cpu() for t in toks])
    tiny.assert_logits_close(step, ref, dtype, "four tokens one by one")
    two = torch.cat([runner.step([StepEntry("t", toks[:2], [0, 1])]).float().cpu(),
                     runner.step([StepEntry("t", toks[2:], [0, 1])]).float().cpu()])
    tiny.assert_logits_close(two, ref, dtype, "two and two")


@pytest.mark.parametrize("dtype", DTYPES)
def test_pipelined_steps_match_synchronous_ones(folders, dtype):
    """Launching a step before the tokens of the one before it have been read back changes
    nothing: same tokens, a stop token ends a request at the same place, pages all come back."""
    from hipinfer_b200 import Engine

    folder, cfg, w = folders["c"]
    prompts = [tiny.random_tokens(n, cfg["vocab_size"], 90 + i) for i, n in enumerate((40, 3, 70, 21, 9))]
    outs = {}
    for pipeline in (False, True):
        eng = Engine(folder, dtype=dtype, max_batch=3, max_seq=256, max_prefill=32, num_pages=20, pipeline=pipeline)
        free = eng.generate(prompts, 25, temperature=0.7, seed=3)
        stop = free[0][7]                                   # a token the first request produces on the way
        ids = [eng.add_request(p, 25, temperature=0.7, seed=3, stop_token_ids=[stop]) for p in prompts]
        res = eng.run()
        outs[pipeline] = (free, [res[i] for i in ids])
        eng.runner.cache.check()
        assert eng.runner.cache.free_pages() == [20] and eng.runner.cache.slots.free_count == 3
        eng.close()
        first = res[ids[0]]
        assert first[-1] == stop and stop not in first[:-1] and len(first) <= 8
        for i, f in zip(ids, free):                          # a stopped request is a prefix of the free one
            assert res[i] == f[:len(res[i])] and (len(res[i]) == 25 or res[i][-1] == stop)
    assert outs[False] == outs[True]


def test_slot_calls_and_bad_arguments(folders):
    """prefill / decode / history / logits / prefill_logits as in the reference's binding
    (scripts/hipinfer.py:392-440), and ValueError for bad arguments (386-390)."""
    folder, cfg, w = folders["a"]
    eng = engine(folder, "float32", max_batch=2, max_seq=64, max_prefill=8)
    p0, p1 = tiny.random_tokens(11, 256, 1), tiny.random_tokens(5, 256, 2)
    want0, _ = plain.generate_greedy(cfg, w, p0, 6)
    want1, _ = plain.generate_greedy(cfg, w, p1, 6)
    assert eng.prefill(0, p0) == want0[0] and eng.prefill(1, p1) == want1[0]
    ms = eng.decode(2, 5)
    assert ms > 0
    assert eng.history(0, len(p0), 6) == want0 and eng.history(1, len(p1), 6) == want1
    assert eng.history(0, 0, len(p0)) == p0
    lg = eng.logits(2)
    assert lg.shape == (2, 256)
    ref = plain.forward(cfg, w, p0 + want0[:5])[-1]
    assert float((lg[0].cpu() - ref).abs().max()) < 2e-5 * float(ref.abs().max())
    allp = eng.prefill_logits(0, p0)                      # p0 = 0 starts the slot afresh
    tiny.assert_logits_close(allp.cpu(), plain.forward(cfg, w, p0), "float32", "prefill_logits")
    more = eng.prefill_logits(0, want0[:2], p0=len(p0))   # and a later call continues it
    tiny.assert_logits_close(more.cpu(), plain.forward(cfg, w, p0 + want0[:2])[len(p0):], "float32", "continued")
    for bad in (lambda: eng.prefill(2, p0), lambda: eng.prefill(0, [256]), lambda: eng.prefill(0, []),
                lambda: eng.prefill(0, [1] * 65), lambda: eng.prefill(0, [1, 2], p0=3), lambda: eng.decode(3, 1),
                lambda: eng.history(0, 0, 1000), lambda: eng.generate([1, 2, 999], 2),
                lambda: eng.generate([1] * 60, 10)):
        with pytest.raises(ValueError):
            bad()
    assert (eng.vocab, eng.hidden, eng.inter, eng.layers, eng.heads, eng.kv_heads, eng.head_dim, eng.tied) == \
        (256, 64, 128, 2, 4, 2, 16, True)
    assert eng.kv_bytes_per_token == 2 * 2 * 2 * 16 * 4 and eng.weight_bytes > 0
    eng.close()


def test_smoke_entry_point():
    import __graft_entry__ as entry

    entry.smoke()


# ------------------------------------------------------------------------------------------
# a kernel that gave up on a bounded wait is an error of the step, not silent wrong tokens
# ------------------------------------------------------------------------------------------
def test_a_wait_that_runs_out_returns_and_raises(folders):
    """The one kernel whose wait cannot complete (its barrier expects bytes that nothing brings) gives up after
    a few thousand polls: the launch returns, the status word is 1, the host raises KernelTimeout and clears it,
    the block's tensor memory was freed (the tensor-core kernels run right afterwards), and the engine's
    own entry points raise where they next wait for the device."""
    from hipinfer_b200.kernels import fast, ops

    fast.check_status()
    out = fast.wait_selftest(polls=3000)
    torch.cuda.synchronize()
    assert out.tolist() == [0, 1], "the wait cannot have completed, and the abort flag must be up"
    assert int(fast.status_word()[0]) == 1
    with pytest.raises(fast.KernelTimeout):
        ops.check_device_status()
    assert int(fast.status_word()[0]) == 0
    ops.check_device_status()                      # cleared: no second error
    # the tensor-core product afterwards (it allocates all of its block's tensor memory) is right
    g = torch.Generator(device="cuda").manual_seed(0)
    a = (torch.randn(256, 512, generator=g, device="cuda") * 0.5).bfloat16()
    w = (torch.randn(384, 512, generator=g, device="cuda") * 0.5).bfloat16()
    got = torch.empty(256, 384, dtype=torch.float32, device="cuda")
    for _ in range(4):
        fast.gemm_tc(a, w, got, fast.EPI_F32)
    torch.cuda.synchronize()
    ops.check_device_status()
    assert torch.allclose(got, a.float() @ w.float().t(), rtol=1e-3, atol=1e-2)
    # through the engine: the word raised by a kernel of a step ends generation with the error
    folder, cfg, weights = folders["c"]
    prompt = tiny.random_tokens(40, cfg["vocab_size"], 3)
    for pipeline in (True, False):
        eng = engine(folder, "bfloat16", max_batch=2, max_seq=128, pipeline=pipeline)
        fast.wait_selftest(polls=2000)
        with pytest.raises(fast.KernelTimeout):
            eng.generate(prompt, 4)
        eng.close()
    want, steps = plain.generate_greedy(cfg, weights, prompt, 4)
    eng = engine(folder, "bfloat16", max_batch=2, max_seq=128)
    check_tokens(eng.generate(prompt, 4), want, steps, "bfloat16", "after a timeout")
    eng.close()


def test_replay_ends_with_the_error(folders, tmp_path, monkeypatch):
    """trace_run's loop: a status word raised during a step ends the replay with KernelTimeout."""
    import io
    import json

    from hipinfer_b200.engine import replay
    from hipinfer_b200.kernels import fast

    folder, cfg, _ = folders["c"]
    fast.check_status()
    fast.status_word()[0] = 1                  # as a kernel's give-up path would leave it
    monkeypatch.setattr("sys.stdin", io.StringIO(json.dumps({"step": 0, "entries": [{"id": "a", "tokens": [1, 2, 3], "want": [2]}]}) + "\n"))
    with pytest.raises(fast.KernelTimeout):
        replay.main(["--model", folder, "--dtype", "bfloat16", "--out", str(tmp_path), "--max-tokens", "64"])
    assert int(fast.status_word()[0]) == 0
