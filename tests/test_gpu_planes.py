"""The named planes that a dumped step leaves (hipinfer_b200/parts/planes.py): every plane of every layer against the
plain implementation's parts, for a whole prompt and for decoded tokens, in 32-bit and in bfloat16; that a dumped step
returns the logits of an ordinary one; and that a fault planted in one weight of one layer is found at that layer's
sub-step and not before."""
import pytest
import torch

import plain_llama as plain
import tiny

pytestmark = pytest.mark.gpu


def plain_planes(cfg, w, tokens):
    """The same planes from the plain parts: {(layer, name): [T, ...]} for a whole sequence."""
    T = len(tokens)
    pos = list(range(T))
    D, Hq, Hkv = plain.head_dim_of(cfg), cfg["num_attention_heads"], plain.kv_heads_of(cfg)
    eps = cfg["rms_norm_eps"]
    inv = plain.rope_inv_freq(D, cfg["rope_theta"], cfg.get("rope_scaling"))
    cos, sin = plain.rope_cos_sin(pos, inv)
    out = {}
    x = plain.embed(tokens, w["model.embed_tokens.weight"])
    out[(-1, "embedding")] = x
    for l in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{l}."
        xn = plain.rmsnorm(x, w[p + "input_layernorm.weight"], eps)
        out[(l, "mixer_norm")] = xn
        q = plain.apply_rope((xn @ w[p + "self_attn.q_proj.weight"].T).reshape(T, Hq, D), cos, sin)
        k = plain.apply_rope((xn @ w[p + "self_attn.k_proj.weight"].T).reshape(T, Hkv, D), cos, sin)
        v = (xn @ w[p + "self_attn.v_proj.weight"].T).reshape(T, Hkv, D)
        out[(l, "q")] = q.reshape(T, Hq * D)
        att = plain.attention_scores_softmax_values(q, k, v, pos, pos).reshape(T, Hq * D)
        out[(l, "attention")] = att
        x = x + att @ w[p + "self_attn.o_proj.weight"].T
        out[(l, "after_mixer")] = x
        xn = plain.rmsnorm(x, w[p + "post_attention_layernorm.weight"], eps)
        out[(l, "feed_forward_norm")] = xn
        g, u = xn @ w[p + "mlp.gate_proj.weight"].T, xn @ w[p + "mlp.up_proj.weight"].T
        act = (g / (1.0 + torch.exp(-g))) * u
        out[(l, "activation")] = act
        x = x + act @ w[p + "mlp.down_proj.weight"].T
        out[(l, "after_feed_forward")] = x
    return out


def rows(planes_, lo, hi):
    return {k: v[lo:hi] for k, v in planes_.items()}


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    out = {}
    for which in ("b", "c"):
        f = tiny.make_model_folder(tmp_path_factory.mktemp(f"planes_{which}"), which, torch.bfloat16)
        out[which] = (f,) + plain.read_model(f)
    return out


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("which", ["b", "c"])
def test_every_plane_of_a_prompt_and_of_decoded_tokens(models, which, dtype):
    from hipinfer_b200.engine import ModelRunner, StepEntry
    from hipinfer_b200.parts import planes

    folder, cfg, w = models[which]
    toks = tiny.random_tokens(90, cfg["vocab_size"], 3)
    want = plain_planes(cfg, w, toks)
    ref_logits = plain.forward(cfg, w, toks)
    runner = ModelRunner.from_folder(folder, dtype=dtype, max_model_len=128, max_num_seqs=2)
    tol = 2e-5 if dtype == "float32" else 3e-2
    got = {}
    logits = runner.step([StepEntry("r", toks[:80], [79])], dump=got)
    names = {k[1] for k in got}
    assert names == set(planes.PLANES) | {"embedding"} and len(got) == 1 + cfg["num_hidden_layers"] * len(planes.PLANES)
    assert planes.first_difference(got, rows(want, 0, 80), tol) is None
    tiny.assert_logits_close(logits.float().cpu(), ref_logits[79:80], dtype, "dumped prompt", group=(f"planes {which}", "prompt"))
    for t in range(80, 90):                       # decoded tokens: dumped steps beside graph-replayed ones
        got = {}
        dumped = runner.step([StepEntry("r", [toks[t]], [0])], dump=got if t % 2 == 0 else None)
        tiny.assert_logits_close(dumped.float().cpu(), ref_logits[t:t + 1], dtype, f"decode {t}", group=(f"planes {which}", "decode"))
        if t % 2 == 0:
            assert planes.first_difference(got, rows(want, t, t + 1), tol) is None
        else:
            assert got == {}
    runner.end("r")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_planted_fault_is_found_at_its_sub_step(models, dtype, tmp_path):
    """One row of layer 1's up projection is scaled in the engine's copy of the weights: every plane up to layer 1's
    feed-forward norm agrees with the plain implementation of the untouched weights, "activation" of layer 1 is the
    first that does not. The same with a fault in layer 0's output projection: "attention" still agrees, "after_mixer"
    is the first."""
    import os
    import shutil

    from safetensors.torch import load_file, save_file

    from hipinfer_b200.engine import ModelRunner, StepEntry
    from hipinfer_b200.parts import planes

    folder, cfg, w = models["b"]
    toks = tiny.random_tokens(40, cfg["vocab_size"], 9)
    want = plain_planes(cfg, w, toks)
    tol = 2e-5 if dtype == "float32" else 3e-2
    for name, first in (("model.layers.1.mlp.up_proj.weight", (1, "activation")),
                        ("model.layers.0.self_attn.o_proj.weight", (0, "after_mixer"))):
        bad = tmp_path / name.replace(".", "_")
        shutil.copytree(folder, bad)
        tensors = load_file(os.path.join(bad, "model.safetensors"))
        t = tensors[name].clone()
        t[5] = t[5] * 8.0
        tensors[name] = t
        save_file(tensors, os.path.join(bad, "model.safetensors"))
        runner = ModelRunner.from_folder(str(bad), dtype=dtype, max_model_len=64, max_num_seqs=1)
        got = {}
        runner.step([StepEntry("r", toks, [])], dump=got)
        found = planes.first_difference(got, want, tol)
        assert found is not None and found[0] == first, found
        runner.end("r")


def test_trace_run_writes_the_planes(models, tmp_path):
    from safetensors.torch import load_file

    folder, cfg, w = models["c"]
    toks = tiny.random_tokens(20, cfg["vocab_size"], 4)
    want = plain_planes(cfg, w, toks)
    tr = tiny.TraceRun(folder, "float32", tmp_path, 64, extra=("--planes",))
    tr.step([("r", toks[:18], [])])
    logits = tr.step([("r", toks[18:], [1])], end=["r"])
    tr.close()
    tiny.assert_logits_close(logits, plain.forward(cfg, w, toks)[19:20], "float32", "trace_run --planes", group=("planes c", "trace_run"))
    from hipinfer_b200.parts import planes

    for step, (lo, hi) in enumerate(((0, 18), (18, 20))):
        file = load_file(str(tmp_path / f"{step}.planes.safetensors"))
        got = {(int(k.split(".", 1)[0]), k.split(".", 1)[1]): v for k, v in file.items()}
        assert len(got) == 1 + cfg["num_hidden_layers"] * len(planes.PLANES)
        assert planes.first_difference(got, rows(want, lo, hi), 2e-5) is None
