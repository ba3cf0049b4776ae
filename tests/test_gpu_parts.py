"""Each part alone beside the plain implementation, and the generality of the assembly: toy
parts and a toy architecture that are defined HERE and registered through the public
registries, without a change to the framework's files: a mixer with state of its own, a window
of keys, a layer that runs twice, a layer that reads another layer's cache."""
import math
from dataclasses import dataclass

import pytest
import torch

import plain_llama as plain
import tiny

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DT = [torch.float32, torch.bfloat16]


def ctx_for(dtype, page_size=16, max_len=256):
    from hipinfer_b200.parts import BuildContext

    return BuildContext(dtype, torch.device(DEV), page_size, max_len)


def rnd(*shape, seed=0, scale=1.0, dtype=torch.float32):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(dtype)


class FakeBatch:
    """What a part sees of a step, for one request of n tokens starting at position ctx."""

    def __init__(self, n, ctx, block_table, page_size):
        i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
        pos = list(range(ctx, ctx + n))
        self.n_rows, self.n_requests, self.n_want = n, 1, 0
        self.positions, self.row_request = i32(pos), i32([0] * n)
        self.req_q_start, self.req_q_len, self.req_ctx_len, self.req_state_slot = i32([0]), i32([n]), i32([ctx]), i32([0])
        self.block_tables = [i32([block_table])]
        self.slot_maps = [i32([block_table[p // page_size] * page_size + p % page_size for p in pos])]
        self.h_q_start, self.h_q_len, self.h_ctx_len, self.h_state_slot = [0], [n], [ctx], [0]
        self.max_pos, self.max_q_len = ctx + n - 1, n


@pytest.mark.parametrize("dtype", DT)
def test_rmsnorm_part(dtype):
    from hipinfer_b200.parts import PartSpec, build_part

    part = build_part("norm", PartSpec("rmsnorm", dict(name="n.weight", size=200, eps=1e-3)), ctx_for(dtype), "p.")
    assert [(s.name, s.shape, s.init) for s in part.param_specs()] == [("p.n.weight", (200,), "ones")]
    w = 1 + rnd(200, seed=1) * 0.1
    part.load({"p.n.weight": w.to(torch.bfloat16).to(DEV)})
    x = rnd(9, 200, seed=2, scale=2.0).to(DEV)
    ref = plain.rmsnorm(x.cpu(), w.to(torch.bfloat16).float(), 1e-3)
    tol = 1e-5 if dtype == torch.float32 else 1e-2
    torch.testing.assert_close(part.forward(x).float().cpu(), ref, rtol=tol, atol=tol)


@pytest.mark.parametrize("dtype", DT)
def test_swiglu_part(dtype):
    from hipinfer_b200.parts import PartSpec, build_part

    H, I, T = 72, 176, 21
    part = build_part("feed_forward", PartSpec("swiglu", dict(hidden_size=H, intermediate_size=I)), ctx_for(dtype), "l.")
    assert sorted(s.name for s in part.param_specs()) == ["l.mlp.down_proj.weight", "l.mlp.gate_proj.weight", "l.mlp.up_proj.weight"]
    wt = {n: rnd(*shape, seed=i, scale=0.1, dtype=torch.bfloat16) for i, (n, shape) in enumerate(
        [("l.mlp.gate_proj.weight", (I, H)), ("l.mlp.up_proj.weight", (I, H)), ("l.mlp.down_proj.weight", (H, I))])}
    part.load({k: v.to(DEV) for k, v in wt.items()})
    xn = rnd(T, H, seed=5).to(dtype)
    x = rnd(T, H, seed=6)
    want = x + plain.swiglu_mlp(xn.float(), *(wt[f"l.mlp.{k}_proj.weight"].float() for k in ("gate", "up", "down")))
    xd = x.to(DEV)
    left = part.forward(xn.to(DEV), xd, None)
    if left is not None:            # a few bfloat16 rows: the last sum is left to the next reader of x
        assert left.out is xd and left.accumulate
        left.finish()
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    torch.testing.assert_close(xd.cpu(), want, rtol=tol, atol=tol)
    with pytest.raises(ValueError, match="multiple of 16"):
        build_part("feed_forward", PartSpec("swiglu", dict(hidden_size=H, intermediate_size=100)), ctx_for(dtype), "l.")


@pytest.mark.parametrize("dtype", DT)
@pytest.mark.parametrize("Hq,Hkv,D,window,scaling", [(4, 2, 16, 0, None), (6, 2, 64, 0, "llama3"), (3, 1, 32, 24, None)])
def test_attention_mixer_alone(dtype, Hq, Hkv, D, window, scaling):
    """The attention part on a cache it fills itself: 50 tokens whole, against 37 then 13."""
    from hipinfer_b200.cache import CacheGroupSpec, CacheStorage
    from hipinfer_b200.models.decoder import StepCachePlan
    from hipinfer_b200.parts import PartSpec, build_part

    H, ps, n = 80, 16, 50
    sc = dict(rope_type="llama3", factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0,
              original_max_position_embeddings=32) if scaling else None
    pos_spec = PartSpec("rope", dict(head_dim=D, theta=10000.0, scaling=sc))
    ctx = ctx_for(dtype, ps, 128)
    part = build_part("mixer", PartSpec("attention", dict(hidden_size=H, n_heads=Hq, n_kv_heads=Hkv, head_dim=D,
                                                          window=window, position=pos_spec)), ctx, "l.")
    need = part.cache_need()
    assert (need.kind, need.kv_heads, need.head_dim, need.window) == ("window" if window else "full", Hkv, D, window)
    names = {k: f"l.self_attn.{k}_proj.weight" for k in "qkvo"}
    shapes = {"q": (Hq * D, H), "k": (Hkv * D, H), "v": (Hkv * D, H), "o": (H, Hq * D)}
    wt = {names[k]: rnd(*shapes[k], seed=i, scale=0.15, dtype=torch.bfloat16) for i, k in enumerate("qkvo")}
    part.load({k: v.to(DEV) for k, v in wt.items()})
    xn = rnd(n, H, seed=9).to(dtype)
    x0 = rnd(n, H, seed=10)
    inv = plain.rope_inv_freq(D, 10000.0, sc)
    want = x0 + plain.attention_block(xn.float(), *(wt[names[k]].float() for k in "qkvo"), list(range(n)), Hq, Hkv, D, inv,
                                      window or None)
    table = [5, 2, 7, 0]                                     # pages in no particular order
    # the error is measured against the size of what the mixer adds: 32-bit rounding, or a few roundings to
    # 8 bits of mantissa (q, k, v, the probabilities and the attention output)
    scale = float((want - x0).abs().max())
    tol = (2e-5 if dtype == torch.float32 else 2e-2) * scale
    for cuts in ([n], [37, 13]):
        storage = CacheStorage([CacheGroupSpec("g", need.kind, 1, Hkv, D, window)], [8], ps, dtype, DEV, {}, 1)
        cache = storage.layer_cache(StepCachePlan(0, 0, True))
        x = x0.clone().to(DEV)
        done = 0
        for c in cuts:
            left = part.forward(xn[done:done + c].to(DEV), x[done:done + c], FakeBatch(c, done, table, ps), cache, {})
            if left is not None:
                left.finish()
            done += c
        err = float((x.cpu() - want).abs().max())
        assert err <= tol, f"cuts {cuts}: max |diff| {err:.3e} > {tol:.3e} (scale {scale:.3e})"


@pytest.mark.parametrize("dtype", DT)
def test_embedding_and_head_parts(dtype):
    from hipinfer_b200.parts import PartSpec, build_part

    V, H = 301, 72
    emb = build_part("embedding", PartSpec("token", dict(name="e.weight", vocab_size=V, hidden_size=H)), ctx_for(dtype))
    tied = build_part("head", PartSpec("linear", dict(tied_to="e.weight", vocab_size=V, hidden_size=H)), ctx_for(dtype))
    own = build_part("head", PartSpec("linear", dict(name="h.weight", vocab_size=V, hidden_size=H)), ctx_for(dtype))
    assert tied.param_specs() == [] and [s.name for s in own.param_specs()] == ["h.weight"]
    e, h = rnd(V, H, seed=1, dtype=torch.bfloat16), rnd(V, H, seed=2, dtype=torch.bfloat16)
    tensors = {"e.weight": e.to(DEV), "h.weight": h.to(DEV)}
    for p in (emb, tied, own):
        p.load(tensors)
    tok = torch.tensor([0, 300, 17], dtype=torch.int32, device=DEV)
    assert torch.equal(emb.forward(tok).cpu(), e.float()[[0, 300, 17]])
    xn = rnd(3, H, seed=3).to(dtype)
    tol = 1e-5 if dtype == torch.float32 else 1e-2
    torch.testing.assert_close(tied.forward(xn.to(DEV)).cpu(), xn.float() @ e.float().T, rtol=tol, atol=tol)
    torch.testing.assert_close(own.forward(xn.to(DEV)).cpu(), xn.float() @ h.float().T, rtol=tol, atol=tol)


# ------------------------------------------------------------------------------------------
# A toy architecture, defined and registered here: nothing in the framework's files knows it.
#   layer 0: attention (all keys) + SwiGLU          layer 1: DecayMixer (state of its own) + SwiGLU
#   layer 2: attention with a window + SwiGLU
#   order:   0, 1, 2, 1 again (its own state), 0 again reading the cache the first step wrote
# ------------------------------------------------------------------------------------------
def _register_toy():
    from hipinfer_b200.config import ModelConfig, register_architecture, take
    from hipinfer_b200.parts import LayerSpec, Mixer, ModelSpec, PartSpec, RunStep, register_part
    from hipinfer_b200.weights import ParamSpec

    class DecayMixer(Mixer):
        """h_t = a h_{t-1} + xn_t per request, carried from step to step in the request's state
        slot; the mixer's output is h_t W^T. It keeps no keys or values."""

        def __init__(self, params, ctx, prefix=""):
            super().__init__(params, ctx, prefix)
            self.hidden, self.a, self.name = params["hidden_size"], params["decay"], prefix + "decay.weight"

        def param_specs(self):
            return [ParamSpec(self.name, (self.hidden, self.hidden))]

        def load(self, tensors):
            self.w = tensors[self.name].float()

        def state_need(self):
            return {"h": ((self.hidden,), torch.float32)}

        def forward(self, xn, x, batch, cache, state):
            """Indexed with the batch's DEVICE arrays only (row -> request, first row, rows and state slot of a
            request), with no loop over requests on the host: the same code is recorded into the CUDA graph of
            decode-only steps and replayed with other requests in the rows."""
            assert cache is None
            T = xn.shape[0]
            req = batch.row_request.long()
            t = torch.arange(T, device=xn.device)
            j = t - batch.req_q_start.long()[req]                       # a row's place within its request's rows
            slots = batch.req_state_slot.long()
            same = req[:, None] == req[None, :]
            lag = (t[:, None] - t[None, :]).clamp(min=0).float()
            mix = torch.where(same & (t[:, None] >= t[None, :]), self.a ** lag, torch.zeros((), device=xn.device))
            h = mix @ xn.float() + (self.a ** (j + 1).float())[:, None] * state["h"][slots[req]]
            x += h @ self.w.T
            last = batch.req_q_start.long() + batch.req_q_len.long() - 1
            state["h"][slots] = h[last]

    @dataclass(frozen=True)
    class ToyConfig(ModelConfig):
        vocab_size: int
        hidden_size: int
        n_heads: int
        n_kv_heads: int
        head_dim: int
        intermediate_size: int
        window: int
        decay: float
        eps: float

        @classmethod
        def from_dict(cls, d):
            return cls(d["architectures"][0], *(take(d, k, int) for k in ("vocab_size", "hidden_size", "n_heads",
                       "n_kv_heads", "head_dim", "intermediate_size", "window")), take(d, "decay", float), take(d, "eps", float))

        def to_dict(self):
            return dict(architectures=[self.architecture], **{k: getattr(self, k) for k in (
                "vocab_size", "hidden_size", "n_heads", "n_kv_heads", "head_dim", "intermediate_size", "window", "decay", "eps")})

    def toy_spec(c):
        H = c.hidden_size
        norm = lambda name: PartSpec("rmsnorm", dict(name=name, size=H, eps=c.eps))
        ffn = PartSpec("swiglu", dict(hidden_size=H, intermediate_size=c.intermediate_size))
        pos = PartSpec("rope", dict(head_dim=c.head_dim, theta=10000.0, scaling=None))
        att = lambda window: PartSpec("attention", dict(hidden_size=H, n_heads=c.n_heads, n_kv_heads=c.n_kv_heads,
                                                        head_dim=c.head_dim, window=window, position=pos))
        mixers = [att(0), PartSpec("toy_decay", dict(hidden_size=H, decay=c.decay)), att(c.window)]
        layers = tuple(LayerSpec(f"toy.layers.{i}.", "pre_norm", dict(
            mixer=m, mixer_norm=norm("input_layernorm.weight"), feed_forward=ffn,
            feed_forward_norm=norm("post_attention_layernorm.weight"))) for i, m in enumerate(mixers))
        order = (RunStep(0), RunStep(1), RunStep(2), RunStep(1), RunStep(0, reads_cache_of=0))
        return ModelSpec(c.architecture, H, c.vocab_size, 256,
                         PartSpec("token", dict(name="toy.embed.weight", vocab_size=c.vocab_size, hidden_size=H)), layers, order,
                         norm("toy.norm.weight"), PartSpec("linear", dict(tied_to="toy.embed.weight", vocab_size=c.vocab_size,
                                                                         hidden_size=H)))

    register_part("mixer", "toy_decay", DecayMixer)
    register_architecture("ToyForCausalLM", ToyConfig, toy_spec)


TOY = dict(architectures=["ToyForCausalLM"], vocab_size=200, hidden_size=64, n_heads=4, n_kv_heads=2, head_dim=32,
           intermediate_size=96, window=40, decay=0.5, eps=1e-5)


def toy_plain(c, w, tokens):
    """The toy model on a whole sequence with the plain implementation's parts."""
    T, H, Hq, Hkv, D = len(tokens), c["hidden_size"], c["n_heads"], c["n_kv_heads"], c["head_dim"]
    pos = list(range(T))
    inv = plain.rope_inv_freq(D, 10000.0)
    x = plain.embed(tokens, w["toy.embed.weight"])

    def norms(i):
        p = f"toy.layers.{i}."
        return w[p + "input_layernorm.weight"], w[p + "post_attention_layernorm.weight"]

    def mlp(i, x):
        p = f"toy.layers.{i}.mlp."
        return x + plain.swiglu_mlp(plain.rmsnorm(x, norms(i)[1], c["eps"]), w[p + "gate_proj.weight"], w[p + "up_proj.weight"],
                                    w[p + "down_proj.weight"])

    def qkvo(i):
        return [w[f"toy.layers.{i}.self_attn.{k}_proj.weight"] for k in "qkvo"]

    def decay(x):
        xn, h, out = plain.rmsnorm(x, norms(1)[0], c["eps"]), torch.zeros(H), []
        for t in range(T):
            h = c["decay"] * h + xn[t]
            out.append(h @ w["toy.layers.1.decay.weight"].T)
        return mlp(1, x + torch.stack(out))

    xn0 = plain.rmsnorm(x, norms(0)[0], c["eps"])
    x = mlp(0, x + plain.attention_block(xn0, *qkvo(0), pos, Hq, Hkv, D, inv))
    x = decay(x)
    x = mlp(2, x + plain.attention_block(plain.rmsnorm(x, norms(2)[0], c["eps"]), *qkvo(2), pos, Hq, Hkv, D, inv, c["window"]))
    x = decay(x)
    # layer 0 again: queries from here, keys and values as the first step stored them
    wq, wk, wv, wo = qkvo(0)
    cos, sin = plain.rope_cos_sin(pos, inv)
    k0 = plain.apply_rope((xn0 @ wk.T).reshape(T, Hkv, D), cos, sin)
    v0 = (xn0 @ wv.T).reshape(T, Hkv, D)
    q = plain.apply_rope((plain.rmsnorm(x, norms(0)[0], c["eps"]) @ wq.T).reshape(T, Hq, D), cos, sin)
    x = mlp(0, x + plain.attention_scores_softmax_values(q, k0, v0, pos, pos).reshape(T, Hq * D) @ wo.T)
    return plain.lm_head(x, w["toy.norm.weight"], w["toy.embed.weight"], c["eps"])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_architecture_registered_from_the_test(dtype):
    from hipinfer_b200.config import config_from_dict, get_architecture
    from hipinfer_b200.engine import ModelRunner
    from hipinfer_b200.parts import spec_param_specs
    from hipinfer_b200.weights import random_weights

    _register_toy()
    cfg = config_from_dict(TOY)
    spec = get_architecture("ToyForCausalLM").build_spec(cfg)
    tensors = random_weights(spec_param_specs(spec), seed=9, std=0.08, norm_std=0.1, dtype=torch.bfloat16)
    assert "toy.layers.1.decay.weight" in tensors and "toy.layers.1.self_attn.q_proj.weight" not in tensors
    runner = ModelRunner(cfg, {k: v.to(DEV) for k, v in tensors.items()}, dtype=dtype, num_pages=40, max_model_len=256,
                         max_num_seqs=4)      # CUDA graphs on: decode-only steps are replayed, the mixer's state with them
    m = runner.model
    assert [(g.kind, g.n_layers, g.window) for g in m.cache_groups] == [("full", 1, 0), ("window", 1, 40)]
    assert [p and (p.group, p.slot, p.write) for p in m.cache_plan] == [(0, 0, True), None, (1, 0, True), None, (0, 0, False)]
    assert sorted(m.state_specs) == [(1, "h"), (3, "h")]                       # the layer that runs twice has two states
    w = {k: v.float() for k, v in tensors.items()}
    requests = {f"t{i}": tiny.random_tokens(n, 200, 60 + i) for i, n in enumerate([150, 33, 90, 64, 7, 120])}
    ref = {rid: toy_plain(TOY, w, toks) for rid, toks in requests.items()}
    st = tiny.RunnerStepper(runner)
    for name, plan in (("whole", tiny.plan_whole(requests)), ("portions", tiny.plan_portions(requests)),
                       ("tail", tiny.plan_tail_decode(requests, 12)), ("mixed", tiny.plan_mixed(requests, 3))):
        got = tiny.run_plan(st, requests, plan)
        for rid in requests:
            tiny.assert_logits_close(got[rid], ref[rid], dtype, f"toy {name} {rid}", group=("toy architecture", name))
        runner.cache.check()
        assert runner.cache.free_pages() == [40, 40] and runner.cache.slots.free_count == 4
    assert runner._graphs, "no decode-only step went through a CUDA graph"
    # the window group gives pages back while a long request is still running; the full group does not
    from hipinfer_b200.engine import StepEntry
    runner.step([StepEntry("long", requests["t0"], [])])
    held = [sum(1 for p in t if p >= 0) for t in runner.cache.get("long").tables]
    assert held == [10, 4]            # 150 tokens fill 10 pages; keys 111..149 are still visible: pages 6..9
    runner.end("long")


# ------------------------------------------------------------------------------------------
# A second toy architecture: a position encoding and a feed-forward of its own kind.
#   layer 0: attention with "toy_decay_position" (no rotation: q_t is scaled by e^(+l t), k_s by e^(-l s), so a
#            score carries the factor e^(l (t - s))) + "toy_top1_experts" (a router picks one of E small experts)
#   layer 1: attention with rope + SwiGLU in a block kind of its own, "toy_sandwich", which has six parts: a norm
#            before AND after the mixer, and before and after the feed-forward
# ------------------------------------------------------------------------------------------
def _register_toy2():
    from hipinfer_b200.config import ModelConfig, register_architecture, take
    from hipinfer_b200.parts import LayerSpec, ModelSpec, Part, PartSpec, RunStep, register_part
    from hipinfer_b200.parts.block import build_slots
    from hipinfer_b200.weights import ParamSpec

    class SandwichBlock(Part):
        """x += post_norm(mixer(pre_norm(x))); x += post_norm(feed_forward(pre_norm(x))). Mixers and feed-forwards add
        into the rows they are given, so each gets rows of zeros, whose norm is then added into x."""

        SLOTS = {"mixer_norm": "norm", "mixer": "mixer", "mixer_post_norm": "norm", "feed_forward_norm": "norm",
                 "feed_forward": "feed_forward", "feed_forward_post_norm": "norm"}

        def __init__(self, params, ctx, prefix=""):
            super().__init__(params, ctx, prefix)
            self.parts = build_slots(self, params["layer"], self.SLOTS, ctx, prefix)

        def param_specs(self):
            return [s for p in self.parts for s in p.param_specs()]

        def load(self, tensors):
            for p in self.parts:
                p.load(tensors)

        def weight_bytes(self):
            return sum(p.weight_bytes() for p in self.parts)

        @staticmethod
        def _done(left):
            if left is not None and hasattr(left, "finish"):
                left.finish()

        def forward(self, x, batch, cache, state):
            y = torch.zeros_like(x)
            self._done(self.mixer.forward(self.mixer_norm.forward(x), y, batch, cache, state))
            x += self.mixer_post_norm.forward(y).float()
            y = torch.zeros_like(x)
            self._done(self.feed_forward.forward(self.feed_forward_norm.forward(x), y, batch))
            x += self.feed_forward_post_norm.forward(y).float()

    class DecayPosition(Part):
        """params: head_dim, rate. It has no `pending` argument: the mixer finishes its product first."""

        def __init__(self, params, ctx, prefix=""):
            super().__init__(params, ctx, prefix)
            self.head_dim, self.rate = params["head_dim"], params["rate"]

        def rotate_and_store(self, qkv, positions, slot_map, q_out, k_cache, v_cache, n_heads, n_kv_heads):
            T, D, ps = qkv.shape[0], self.head_dim, self.ctx.page_size
            p = positions.float()[:, None, None]
            q = qkv[:, :n_heads * D].float().reshape(T, n_heads, D) * torch.exp(self.rate * p)
            k = qkv[:, n_heads * D:(n_heads + n_kv_heads) * D].float().reshape(T, n_kv_heads, D) * torch.exp(-self.rate * p)
            v = qkv[:, (n_heads + n_kv_heads) * D:].float().reshape(T, n_kv_heads, D)
            q_out.copy_(q.reshape(T, n_heads * D).to(q_out.dtype))
            if slot_map is not None:
                page, off = (slot_map // ps).long(), (slot_map % ps).long()
                k_cache[page, :, off] = k.to(k_cache.dtype)
                v_cache[page, :, off] = v.to(v_cache.dtype)
            return q_out

    class Top1Experts(Part):
        """params: hidden_size, inner_size, n_experts. y = p_e W2_e relu(W1_e xn), e = arg max of the router's softmax p."""

        def __init__(self, params, ctx, prefix=""):
            super().__init__(params, ctx, prefix)
            self.H, self.I, self.E = params["hidden_size"], params["inner_size"], params["n_experts"]
            self.names = [prefix + n for n in ("moe.router.weight", "moe.w1", "moe.w2")]

        def param_specs(self):
            return [ParamSpec(self.names[0], (self.E, self.H)), ParamSpec(self.names[1], (self.E * self.I, self.H)),
                    ParamSpec(self.names[2], (self.E * self.H, self.I))]

        def load(self, tensors):
            self.router = tensors[self.names[0]].float()
            self.w1 = tensors[self.names[1]].float().reshape(self.E, self.I, self.H)
            self.w2 = tensors[self.names[2]].float().reshape(self.E, self.H, self.I)

        def forward(self, xn, x, batch):
            xf = xn.float()
            p = torch.softmax(xf @ self.router.T, -1)
            e = p.argmax(-1)
            h = torch.relu(torch.einsum("tih,th->ti", self.w1[e], xf))
            x += p.gather(1, e[:, None]) * torch.einsum("thi,ti->th", self.w2[e], h)

    @dataclass(frozen=True)
    class Toy2Config(ModelConfig):
        vocab_size: int
        hidden_size: int
        n_heads: int
        n_kv_heads: int
        head_dim: int
        intermediate_size: int
        n_experts: int
        rate: float
        eps: float

        @classmethod
        def from_dict(cls, d):
            return cls(d["architectures"][0], *(take(d, k, int) for k in ("vocab_size", "hidden_size", "n_heads", "n_kv_heads",
                       "head_dim", "intermediate_size", "n_experts")), take(d, "rate", float), take(d, "eps", float))

        def to_dict(self):
            return dict(architectures=[self.architecture], **{k: getattr(self, k) for k in (
                "vocab_size", "hidden_size", "n_heads", "n_kv_heads", "head_dim", "intermediate_size", "n_experts", "rate", "eps")})

    def toy2_spec(c):
        H = c.hidden_size
        norm = lambda name: PartSpec("rmsnorm", dict(name=name, size=H, eps=c.eps))
        att = lambda pos: PartSpec("attention", dict(hidden_size=H, n_heads=c.n_heads, n_kv_heads=c.n_kv_heads,
                                                     head_dim=c.head_dim, window=0, position=pos))
        mixers = [att(PartSpec("toy_decay_position", dict(head_dim=c.head_dim, rate=c.rate))),
                  att(PartSpec("rope", dict(head_dim=c.head_dim, theta=10000.0, scaling=None)))]
        ffns = [PartSpec("toy_top1_experts", dict(hidden_size=H, inner_size=c.intermediate_size, n_experts=c.n_experts)),
                PartSpec("swiglu", dict(hidden_size=H, intermediate_size=c.intermediate_size))]
        layers = (LayerSpec("toy2.layers.0.", "pre_norm", dict(
                      mixer=mixers[0], mixer_norm=norm("input_layernorm.weight"), feed_forward=ffns[0],
                      feed_forward_norm=norm("post_attention_layernorm.weight"))),
                  LayerSpec("toy2.layers.1.", "toy_sandwich", dict(
                      mixer=mixers[1], mixer_norm=norm("input_layernorm.weight"), mixer_post_norm=norm("post_mixer_norm.weight"),
                      feed_forward=ffns[1], feed_forward_norm=norm("post_attention_layernorm.weight"),
                      feed_forward_post_norm=norm("post_feed_forward_norm.weight"))))
        return ModelSpec(c.architecture, H, c.vocab_size, 256,
                         PartSpec("token", dict(name="toy2.embed.weight", vocab_size=c.vocab_size, hidden_size=H)), layers,
                         (RunStep(0), RunStep(1)), norm("toy2.norm.weight"),
                         PartSpec("linear", dict(tied_to="toy2.embed.weight", vocab_size=c.vocab_size, hidden_size=H)))

    register_part("block", "toy_sandwich", SandwichBlock)
    register_part("position", "toy_decay_position", DecayPosition)
    register_part("feed_forward", "toy_top1_experts", Top1Experts)
    register_architecture("Toy2ForCausalLM", Toy2Config, toy2_spec)


TOY2 = dict(architectures=["Toy2ForCausalLM"], vocab_size=150, hidden_size=64, n_heads=4, n_kv_heads=2, head_dim=64,
            intermediate_size=48, n_experts=3, rate=0.004, eps=1e-6)


def toy2_plain(c, w, tokens):
    T, H, Hq, Hkv, D, E, I = (len(tokens), c["hidden_size"], c["n_heads"], c["n_kv_heads"], c["head_dim"], c["n_experts"],
                              c["intermediate_size"])
    pos = list(range(T))
    x = plain.embed(tokens, w["toy2.embed.weight"])
    p0, p1 = "toy2.layers.0.", "toy2.layers.1."
    # layer 0: attention with the decaying position factors
    xn = plain.rmsnorm(x, w[p0 + "input_layernorm.weight"], c["eps"])
    t = torch.arange(T, dtype=torch.float32)[:, None, None]
    q = (xn @ w[p0 + "self_attn.q_proj.weight"].T).reshape(T, Hq, D) * torch.exp(c["rate"] * t)
    k = (xn @ w[p0 + "self_attn.k_proj.weight"].T).reshape(T, Hkv, D) * torch.exp(-c["rate"] * t)
    v = (xn @ w[p0 + "self_attn.v_proj.weight"].T).reshape(T, Hkv, D)
    x = x + plain.attention_scores_softmax_values(q, k, v, pos, pos).reshape(T, Hq * D) @ w[p0 + "self_attn.o_proj.weight"].T
    # layer 0: one expert per token
    xn = plain.rmsnorm(x, w[p0 + "post_attention_layernorm.weight"], c["eps"])
    p = torch.softmax(xn @ w[p0 + "moe.router.weight"].T, -1)
    w1, w2 = w[p0 + "moe.w1"].reshape(E, I, H), w[p0 + "moe.w2"].reshape(E, H, I)
    for i in range(T):
        e = int(p[i].argmax())
        x[i] = x[i] + p[i, e] * (w2[e] @ torch.relu(w1[e] @ xn[i]))
    # layer 1: the architecture's own parts, each between two norms
    inv = plain.rope_inv_freq(D, 10000.0)
    y = plain.attention_block(plain.rmsnorm(x, w[p1 + "input_layernorm.weight"], c["eps"]),
                              *(w[p1 + f"self_attn.{n}_proj.weight"] for n in "qkvo"), pos, Hq, Hkv, D, inv)
    x = x + plain.rmsnorm(y, w[p1 + "post_mixer_norm.weight"], c["eps"])
    y = plain.swiglu_mlp(plain.rmsnorm(x, w[p1 + "post_attention_layernorm.weight"], c["eps"]),
                         *(w[p1 + f"mlp.{n}_proj.weight"] for n in ("gate", "up", "down")))
    x = x + plain.rmsnorm(y, w[p1 + "post_feed_forward_norm.weight"], c["eps"])
    return plain.lm_head(x, w["toy2.norm.weight"], w["toy2.embed.weight"], c["eps"])


def test_toy_position_encoding_and_routed_feed_forward():
    """Another position encoding and a feed-forward with routing, defined here, in one model beside the
    architecture's own parts (32-bit: a router's arg max is not stable under bfloat16 rounding)."""
    from hipinfer_b200.config import config_from_dict, get_architecture
    from hipinfer_b200.engine import ModelRunner
    from hipinfer_b200.parts import spec_param_specs
    from hipinfer_b200.weights import random_weights

    _register_toy2()
    cfg = config_from_dict(TOY2)
    spec = get_architecture("Toy2ForCausalLM").build_spec(cfg)
    tensors = random_weights(spec_param_specs(spec), seed=11, std=0.08, norm_std=0.1, dtype=torch.float32)
    assert "toy2.layers.0.moe.router.weight" in tensors and "toy2.layers.0.mlp.gate_proj.weight" not in tensors
    assert "toy2.layers.1.post_mixer_norm.weight" in tensors and "toy2.layers.0.post_mixer_norm.weight" not in tensors
    runner = ModelRunner(cfg, {k: v.to(DEV) for k, v in tensors.items()}, dtype="float32", num_pages=30, max_model_len=256,
                         max_num_seqs=4, cuda_graphs=False)
    w = {k: v.float() for k, v in tensors.items()}
    requests = {f"u{i}": tiny.random_tokens(n, 150, 80 + i) for i, n in enumerate([120, 33, 70, 9])}
    ref = {rid: toy2_plain(TOY2, w, toks) for rid, toks in requests.items()}
    st = tiny.RunnerStepper(runner)
    for name, plan in (("whole", tiny.plan_whole(requests)), ("portions", tiny.plan_portions(requests)),
                       ("mixed", tiny.plan_mixed(requests, 3))):
        got = tiny.run_plan(st, requests, plan)
        for rid in requests:
            tiny.assert_logits_close(got[rid], ref[rid], "float32", f"toy2 {name} {rid}", group=("toy architecture 2", name))
        runner.cache.check()
        assert runner.cache.free_pages() == [30] and runner.cache.slots.free_count == 4


# ------------------------------------------------------------------------------------------
# A third toy architecture: a mixer whose cache is not keys and values of one shape, in a group with a retention
# rule of its own. Per token it keeps a latent c (1 x Dc) and two gate vectors g (2 x Dg); a query sees the first
# `sink` tokens and the last `window`; pages wholly between the two are given back while the request runs.
#   layer 0: LatentMixer + SwiGLU      layer 1: attention (all keys) + SwiGLU      order: 0, 1, 0 again (a cache of its own)
# ------------------------------------------------------------------------------------------
def _register_toy3():
    from hipinfer_b200.cache import register_retention
    from hipinfer_b200.config import ModelConfig, register_architecture, take
    from hipinfer_b200.parts import LayerSpec, Mixer, ModelSpec, PartSpec, RunStep, register_part
    from hipinfer_b200.parts.registry import CacheNeed
    from hipinfer_b200.weights import ParamSpec

    def sink_window(spec, q):
        sink = dict(spec.extra)["sink"]
        return ((sink, max(sink, q - spec.window + 1)),)

    register_retention("toy_sink_window", sink_window)

    class LatentMixer(Mixer):
        def __init__(self, params, ctx, prefix=""):
            super().__init__(params, ctx, prefix)
            self.H, self.Dc, self.Dg = params["hidden_size"], params["latent"], params["gate"]
            self.sink, self.window = params["sink"], params["window"]
            self.names = [prefix + f"latent.{n}.weight" for n in ("c", "g", "o")]

        def param_specs(self):
            return [ParamSpec(self.names[0], (self.Dc, self.H)), ParamSpec(self.names[1], (2 * self.Dg, self.H)),
                    ParamSpec(self.names[2], (self.H, self.Dc))]

        def load(self, tensors):
            self.wc, self.wg, self.wo = (tensors[n].float() for n in self.names)

        def cache_need(self):
            return CacheNeed("toy_sink_window", window=self.window, planes=(("c", 1, self.Dc), ("g", 2, self.Dg)),
                             extra=(("sink", self.sink),))

        def forward(self, xn, x, batch, cache, state):
            ps, T = self.ctx.page_size, xn.shape[0]
            C, G = cache.planes["c"], cache.planes["g"]                  # [page, 1, ps, Dc], [page, 2, ps, Dg]
            xf = xn.float()
            c = (xf @ self.wc.T).to(C.dtype)
            g = (xf @ self.wg.T).reshape(T, 2, self.Dg).to(G.dtype)
            if cache.write:
                slot = batch.slot_maps[cache.group].long()
                C[slot // ps, 0, slot % ps] = c
                G[slot // ps, :, slot % ps] = g
            table = batch.block_tables[cache.group].long()               # [R, pages]; -1 where a page was given back
            p = torch.arange(table.shape[1] * ps, device=xn.device)
            page = table[batch.row_request.long()][:, p // ps]           # [T, L]
            pos = batch.positions.long()[:, None]
            visible = (page >= 0) & (p[None] <= pos) & ((p[None] < self.sink) | (p[None] > pos - self.window))
            page, off = page.clamp(min=0), (p % ps)[None].expand_as(page)
            ck, gk = C[page, 0, off].float(), G[page, :, off].float()    # [T, L, Dc], [T, L, 2, Dg]
            score = torch.einsum("td,tld->tl", c.float(), ck) / math.sqrt(self.Dc) + \
                torch.einsum("thd,tlhd->tl", g.float(), gk)
            prob = torch.softmax(score.masked_fill(~visible, float("-inf")), -1)
            x += torch.einsum("tl,tld->td", prob, ck) @ self.wo.T

    @dataclass(frozen=True)
    class Toy3Config(ModelConfig):
        vocab_size: int
        hidden_size: int
        n_heads: int
        n_kv_heads: int
        head_dim: int
        intermediate_size: int
        latent: int
        gate: int
        sink: int
        window: int
        eps: float

        KEYS = ("vocab_size", "hidden_size", "n_heads", "n_kv_heads", "head_dim", "intermediate_size", "latent", "gate",
                "sink", "window")

        @classmethod
        def from_dict(cls, d):
            return cls(d["architectures"][0], *(take(d, k, int) for k in cls.KEYS), take(d, "eps", float))

        def to_dict(self):
            return dict(architectures=[self.architecture], **{k: getattr(self, k) for k in self.KEYS + ("eps",)})

    def toy3_spec(c):
        H = c.hidden_size
        norm = lambda name: PartSpec("rmsnorm", dict(name=name, size=H, eps=c.eps))
        ffn = PartSpec("swiglu", dict(hidden_size=H, intermediate_size=c.intermediate_size))
        mixers = [PartSpec("toy_latent", dict(hidden_size=H, latent=c.latent, gate=c.gate, sink=c.sink, window=c.window)),
                  PartSpec("attention", dict(hidden_size=H, n_heads=c.n_heads, n_kv_heads=c.n_kv_heads, head_dim=c.head_dim, window=0,
                                             position=PartSpec("rope", dict(head_dim=c.head_dim, theta=10000.0, scaling=None))))]
        layers = tuple(LayerSpec(f"toy3.layers.{i}.", "pre_norm", dict(
            mixer=m, mixer_norm=norm("input_layernorm.weight"), feed_forward=ffn,
            feed_forward_norm=norm("post_attention_layernorm.weight"))) for i, m in enumerate(mixers))
        return ModelSpec(c.architecture, H, c.vocab_size, 256,
                         PartSpec("token", dict(name="toy3.embed.weight", vocab_size=c.vocab_size, hidden_size=H)), layers,
                         (RunStep(0), RunStep(1), RunStep(0)), norm("toy3.norm.weight"),
                         PartSpec("linear", dict(tied_to="toy3.embed.weight", vocab_size=c.vocab_size, hidden_size=H)))

    register_part("mixer", "toy_latent", LatentMixer)
    register_architecture("Toy3ForCausalLM", Toy3Config, toy3_spec)


TOY3 = dict(architectures=["Toy3ForCausalLM"], vocab_size=180, hidden_size=80, n_heads=2, n_kv_heads=1, head_dim=32,
            intermediate_size=112, latent=24, gate=8, sink=5, window=40, eps=1e-5)


def toy3_plain(c, w, tokens):
    T, H, Hq, Hkv, D, Dc, Dg = (len(tokens), c["hidden_size"], c["n_heads"], c["n_kv_heads"], c["head_dim"], c["latent"],
                                c["gate"])
    pos = list(range(T))
    t = torch.arange(T)
    visible = (t[None] <= t[:, None]) & ((t[None] < c["sink"]) | (t[None] > t[:, None] - c["window"]))

    def norms(i):
        p = f"toy3.layers.{i}."
        return w[p + "input_layernorm.weight"], w[p + "post_attention_layernorm.weight"]

    def mlp(i, x):
        p = f"toy3.layers.{i}.mlp."
        return x + plain.swiglu_mlp(plain.rmsnorm(x, norms(i)[1], c["eps"]), w[p + "gate_proj.weight"], w[p + "up_proj.weight"],
                                    w[p + "down_proj.weight"])

    def latent(x):
        xn = plain.rmsnorm(x, norms(0)[0], c["eps"])
        lc = xn @ w["toy3.layers.0.latent.c.weight"].T
        lg = (xn @ w["toy3.layers.0.latent.g.weight"].T).reshape(T, 2, Dg)
        score = lc @ lc.T / math.sqrt(Dc) + torch.einsum("thd,shd->ts", lg, lg)
        prob = torch.softmax(score.masked_fill(~visible, float("-inf")), -1)
        return mlp(0, x + (prob @ lc) @ w["toy3.layers.0.latent.o.weight"].T)

    x = latent(plain.embed(tokens, w["toy3.embed.weight"]))
    x = mlp(1, x + plain.attention_block(plain.rmsnorm(x, norms(1)[0], c["eps"]),
                                         *(w[f"toy3.layers.1.self_attn.{k}_proj.weight"] for k in "qkvo"), pos, Hq, Hkv, D,
                                         plain.rope_inv_freq(D, 10000.0)))
    x = latent(x)
    return plain.lm_head(x, w["toy3.norm.weight"], w["toy3.embed.weight"], c["eps"])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_mixer_with_cache_planes_and_a_retention_rule_of_its_own(dtype):
    from hipinfer_b200.config import config_from_dict, get_architecture
    from hipinfer_b200.engine import ModelRunner, StepEntry
    from hipinfer_b200.parts import spec_param_specs
    from hipinfer_b200.weights import random_weights

    _register_toy3()
    cfg = config_from_dict(TOY3)
    spec = get_architecture("Toy3ForCausalLM").build_spec(cfg)
    tensors = random_weights(spec_param_specs(spec), seed=13, std=0.08, norm_std=0.1, dtype=torch.bfloat16)
    runner = ModelRunner(cfg, {k: v.to(DEV) for k, v in tensors.items()}, dtype=dtype, num_pages=40, max_model_len=256,
                         max_num_seqs=4)
    m = runner.model
    assert [(g.kind, g.n_layers, g.planes) for g in m.cache_groups] == \
        [("toy_sink_window", 2, (("c", 1, 24), ("g", 2, 8))), ("full", 1, (("k", 1, 32), ("v", 1, 32)))]
    assert [(p.group, p.slot, p.write) for p in m.cache_plan] == [(0, 0, True), (1, 0, True), (0, 1, True)]
    assert {n: tuple(t.shape) for n, t in runner.storage.kv[0].items()} == {"c": (2, 40, 1, 16, 24), "g": (2, 40, 2, 16, 8)}
    assert runner.storage.bytes_per_token() == (2 * (24 + 16) + 2 * 32) * (4 if dtype == "float32" else 2)
    w = {k: v.float() for k, v in tensors.items()}
    requests = {f"v{i}": tiny.random_tokens(n, 180, 40 + i) for i, n in enumerate([150, 33, 90, 64, 7, 120])}
    ref = {rid: toy3_plain(TOY3, w, toks) for rid, toks in requests.items()}
    st = tiny.RunnerStepper(runner)
    for name, plan in (("whole", tiny.plan_whole(requests)), ("portions", tiny.plan_portions(requests)),
                       ("tail", tiny.plan_tail_decode(requests, 12)), ("mixed", tiny.plan_mixed(requests, 3))):
        got = tiny.run_plan(st, requests, plan)
        for rid in requests:
            tiny.assert_logits_close(got[rid], ref[rid], dtype, f"toy3 {name} {rid}", group=("toy architecture 3", name))
        runner.cache.check()
        assert runner.cache.free_pages() == [40, 40] and runner.cache.slots.free_count == 4
    assert runner._graphs, "no decode-only step went through a CUDA graph"
    # 150 tokens: the latent group keeps page 0 (the first 5 tokens lie on it) and pages 6..9 (tokens 111..149 are
    # still visible to the next query); pages 1..5 went back while the request runs. The attention group keeps all 10.
    runner.step([StepEntry("long", requests["v0"], [])])
    tables = runner.cache.get("long").tables
    assert [i for i, p in enumerate(tables[0]) if p >= 0] == [0, 6, 7, 8, 9] and all(p >= 0 for p in tables[1])
    runner.end("long")


def test_unknown_part_kind_is_named():
    from hipinfer_b200.parts import BuildContext, PartSpec, build_part

    with pytest.raises(KeyError, match="no mixer of kind 'nope'"):
        build_part("mixer", PartSpec("nope", {}), BuildContext.meta())
