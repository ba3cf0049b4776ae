"""One kernel at given sizes, timed with CUDA events: for profiling a kernel alone and for the
roofline figures under `profiles/` (the reference times its kernels one by one the same way,
scripts/bench.py:126-212, and reports GB/s or TFLOP/s from algorithmic bytes and flops).

    python -m hipinfer_b200.kernels.microbench gemm_tc --m 2048 --n 16384 --k 2048 --epi swiglu
    python -m hipinfer_b200.kernels.microbench gemm_stream --m 8 --n 65536 --k 2048
    python -m hipinfer_b200.kernels.microbench attn_decode --batch 64 --context 2176
    python -m hipinfer_b200.kernels.microbench flash_prefill --tokens 2048
    python -m hipinfer_b200.kernels.microbench rmsnorm --m 2048 --n 2048

Between timed launches of kernels whose inputs fit in L2 a buffer larger than L2 is written
(`--flush`, on by default) so that the figures are for operands coming from HBM.
"""
from __future__ import annotations

import argparse
import json
import math
import sys

import torch

EPI = {"f32": 0, "bf16": 1, "add": 2, "swiglu": 3}


def timeit(fn, iters, flush):
    """Median milliseconds of `fn` over `iters` launches, each bracketed by events."""
    scratch = torch.empty(256 << 20, dtype=torch.uint8, device="cuda") if flush else None
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    times = []
    for _ in range(iters):
        if scratch is not None:
            scratch.zero_()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        fn()
        stop.record()
        stop.synchronize()
        times.append(start.elapsed_time(stop))
    times.sort()
    return times[len(times) // 2]


def _prepared(fast, x, nw):
    """A filled NormFeed for residual rows x: what a product with the residual add in its epilogue leaves for the next norm."""
    M, K = x.shape
    feed = fast.NormFeed(nw, 1e-5, M)
    feed.xb.copy_((x * nw.float()).bfloat16())
    feed.ssq.zero_()
    feed.ssq[:, :M] = (x * x).reshape(M, K // 16, 16).sum(-1).T
    feed.filled = True
    return feed


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawTextHelpFormatter)
    ap.add_argument("kernel", choices=["gemm_tc", "gemm_stream", "rows_add", "rows_swiglu", "rows_qkv", "attn_decode", "flash_prefill", "flash_prefill_tc", "rmsnorm"])
    ap.add_argument("--m", type=int, default=8)
    ap.add_argument("--n", type=int, default=16384)
    ap.add_argument("--k", type=int, default=2048)
    ap.add_argument("--epi", default="f32", choices=sorted(EPI))
    ap.add_argument("--tile-n", type=int, default=0)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=2176)
    ap.add_argument("--tokens", type=int, default=2048)
    ap.add_argument("--heads", type=int, default=32)
    ap.add_argument("--kv-heads", type=int, default=8)
    ap.add_argument("--head-dim", type=int, default=64)
    ap.add_argument("--page-size", type=int, default=16)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--no-flush", dest="flush", action="store_false")
    ap.add_argument("--prepared-norm", action="store_true",
                    help="rows_swiglu, rows_qkv: the rows come as a prepared norm (x times the norm's weight and the pieces of "
                         "the sums of squares, as the product before leaves them) instead of the residual rows")
    a = ap.parse_args(argv)

    from . import fast, ops

    dev = "cuda:0"
    g = torch.Generator(device=dev).manual_seed(0)
    rnd = lambda *s: torch.randn(*s, generator=g, device=dev)
    out = {"kernel": a.kernel}
    if a.kernel.startswith("rows"):
        M, N, K = a.m, a.n, a.k
        w = (rnd(N, K) * 0.02).bfloat16()
        nw = torch.ones(K, device=dev, dtype=torch.bfloat16)
        if a.kernel == "rows_add":
            act, acc = rnd(M, K).bfloat16(), torch.zeros(M, N, device=dev)
            fn = lambda: fast.rows_add(act, w, acc)
        elif a.kernel == "rows_swiglu":
            x, act = rnd(M, K), torch.empty(M, N // 2, device=dev, dtype=torch.bfloat16)
            fn = lambda: fast.rows_norm_swiglu(x, nw, 1e-5, w, act, 16)
            if a.prepared_norm:
                feed = _prepared(fast, x, nw)
                fn = lambda: fast.rows_scaled_swiglu(feed, M, w, act, 16)
        else:
            Hq, Hkv, D = a.heads, a.kv_heads, a.head_dim
            N = (Hq + 2 * Hkv) * D
            w = (rnd(N, K) * 0.02).bfloat16()
            x, q = rnd(M, K), torch.empty(M, Hq * D, device=dev, dtype=torch.bfloat16)
            table = ops.rope_table((10000.0 ** (-torch.arange(0, D, 2, dtype=torch.float64) / D)).float().to(dev), 4096)
            pos = torch.arange(M, dtype=torch.int32, device=dev) + 2048
            kc = torch.zeros(M + 4, Hkv, a.page_size, D, device=dev, dtype=torch.bfloat16)
            vc = torch.zeros_like(kc)
            slots = (torch.arange(M, dtype=torch.int32, device=dev) * a.page_size)
            fn = lambda: fast.rows_norm_qkv_rope(x, nw, 1e-5, w, pos, slots, table, q, kc, vc, Hq, Hkv, D, D, a.page_size)
            if a.prepared_norm:
                feed = _prepared(fast, x, nw)
                fn = lambda: fast.rows_scaled_qkv_rope(feed, M, w, pos, slots, table, q, kc, vc, Hq, Hkv, D, D, a.page_size)
        assert fn(), "the rows kernel does not take these sizes"
        ms = timeit(fn, a.iters, a.flush)
        out.update(M=M, N=N, K=K, ms=ms, gbs=N * K * 2 / ms / 1e6)
    elif a.kernel.startswith("gemm"):
        M, N, K, epi = a.m, a.n, a.k, EPI[a.epi]
        x, w = rnd(M, K).bfloat16(), (rnd(N, K) * 0.02).bfloat16()
        c = torch.zeros(M, N // 2 if epi == 3 else N, device=dev, dtype=torch.bfloat16 if epi in (1, 3) else torch.float32)
        if a.kernel == "gemm_tc":
            fn = lambda: fast.gemm_tc(x, w, c, epi, a.tile_n)
        else:
            fn = lambda: fast.gemm_stream(x, w, c, epi)
        ms = timeit(fn, a.iters, a.flush)
        nbytes = N * K * 2 + M * K * 2 + c.numel() * c.element_size()
        out.update(M=M, N=N, K=K, epi=a.epi, ms=ms, tflops=2.0 * M * N * K / ms / 1e9, gbs=nbytes / ms / 1e6)
    elif a.kernel == "rmsnorm":
        x, w = rnd(a.m, a.n), torch.ones(a.n, device=dev, dtype=torch.bfloat16)
        y = torch.empty(a.m, a.n, device=dev, dtype=torch.bfloat16)
        ms = timeit(lambda: ops.rmsnorm(x, w, 1e-5, y), a.iters, a.flush)
        out.update(M=a.m, H=a.n, ms=ms, gbs=a.m * a.n * 6 / ms / 1e6)
    else:
        Hq, Hkv, D, ps = a.heads, a.kv_heads, a.head_dim, a.page_size
        if a.kernel == "attn_decode":
            R, ctx, T = a.batch, a.context, a.batch
            q_len, ctx_len = [1] * R, [ctx - 1] * R
        else:
            R, T, ctx = 1, a.tokens, a.tokens
            q_len, ctx_len = [T], [0]
        pages = -(-ctx // ps)
        kc = (rnd(R * pages, Hkv, ps, D)).bfloat16()
        vc = (rnd(R * pages, Hkv, ps, D)).bfloat16()
        i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)
        bt = torch.arange(R * pages, dtype=torch.int32, device=dev).view(R, pages)
        q = rnd(T, Hq * D).bfloat16()
        o = torch.empty_like(q)
        scale = 1.0 / math.sqrt(D)
        if a.kernel == "attn_decode":
            rr, pos, cl = i32(list(range(R))), i32([ctx - 1] * R), i32(ctx_len)
            fn = lambda: fast.attention_decode(q, kc, vc, bt, None, pos, o, Hq, Hkv, D, ps, 0, scale, ctx - 1, ctx_len=cl)   # row t = request t, as in a decode step
            nbytes = 2 * R * ctx * Hkv * D * 2
            flops = 4.0 * R * ctx * Hq * D
        else:
            qs, ql, cl = i32([0]), i32(q_len), i32(ctx_len)
            impl = fast.flash_prefill_tc if a.kernel == "flash_prefill_tc" else fast.flash_prefill
            fn = lambda: impl(q, kc, vc, bt, qs, ql, cl, o, T, Hq, Hkv, D, ps, 0, scale)
            nbytes = 2 * ctx * Hkv * D * 2 + 2 * T * Hq * D * 2
            flops = 4.0 * Hq * D * (T * (T + 1) / 2)
        ms = timeit(fn, a.iters, a.flush)
        out.update(requests=R, context=ctx, heads=Hq, kv_heads=Hkv, head_dim=D, ms=ms, tflops=flops / ms / 1e9,
                   gbs=nbytes / ms / 1e6)
    torch.cuda.synchronize()
    fast.check_status()
    print(json.dumps({k: (round(v, 4) if isinstance(v, float) else v) for k, v in out.items()}))
    return 0


if __name__ == "__main__":
    sys.exit(main())
