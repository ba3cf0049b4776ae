"""The tensor-core and small-batch bfloat16 kernels, each alone beside a plain float32 statement
of the same operation, at sizes other than the engine's (ragged M, N, K; every tile width)."""
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def rnd(*shape, seed=0, scale=1.0, dtype=torch.bfloat16):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(dtype).to(DEV)


def fast():
    from hipinfer_b200.kernels import fast as f
    return f


def sync_check():
    torch.cuda.synchronize()
    fast().check_status()


SHAPES = [(128, 128, 64), (1, 128, 64), (5, 96, 72), (130, 300, 200), (257, 256, 512), (64, 1000, 320),
          (300, 704, 256), (2048, 512, 2048)]


@pytest.mark.parametrize("tile_n", [128, 192, 256, 512])      # 512: 256 x 256 tiles by CTA pairs
@pytest.mark.parametrize("M,N,K", SHAPES)
def test_gemm_tc_store_and_add(M, N, K, tile_n):
    a, w = rnd(M, K, seed=1), rnd(N, K, seed=2, scale=0.1)
    ref = a.float().double() @ w.float().double().T
    tol = 2e-5 * max(1.0, float(ref.abs().max())) * (K ** 0.5)
    out = torch.full((M + 1, N), 7.0, dtype=torch.float32, device=DEV)
    fast().gemm_tc(a, w, out[:M], fast().EPI_F32, tile_n)
    sync_check()
    assert float((out[:M].double() - ref).abs().max()) < tol
    assert bool((out[M] == 7.0).all()), "wrote past the last row"
    acc = rnd(M, N, seed=3, dtype=torch.float32)
    want = acc.double() + ref
    fast().gemm_tc(a, w, acc, fast().EPI_ADD_F32, tile_n)
    sync_check()
    assert float((acc.double() - want).abs().max()) < tol
    if tile_n == 192:           # the 192-wide tile is for 32-bit results; and a value is the same for every width
        other = torch.empty(M, N, dtype=torch.float32, device=DEV)
        fast().gemm_tc(a, w, other, fast().EPI_F32, 256)
        assert torch.equal(other, out[:M])
        return
    ob = torch.full((M + 1, N), 7.0, dtype=torch.bfloat16, device=DEV)
    if tile_n == 512 and N % 8:     # the pair kernel stores by TMA only: rows of C that are no multiple of 16 bytes are refused
        from hipinfer_b200.kernels.ops import KernelError
        with pytest.raises(KernelError, match="16-byte aligned"):
            fast().gemm_tc(a, w, ob[:M], fast().EPI_BF16, tile_n)
        return
    fast().gemm_tc(a, w, ob[:M], fast().EPI_BF16, tile_n)
    sync_check()
    assert float((ob[:M].double() - ref).abs().max()) < 1e-2 * max(1.0, float(ref.abs().max()))
    assert bool((ob[M] == 7.0).all())


@pytest.mark.parametrize("tile_n", [128, 256, 512])
@pytest.mark.parametrize("M,I,K", [(3, 16, 64), (129, 176, 96), (70, 320, 136), (512, 1024, 256)])
def test_gemm_tc_swiglu(M, I, K, tile_n):
    a = rnd(M, K, seed=4)
    g, u = rnd(I, K, seed=5, scale=0.2), rnd(I, K, seed=6, scale=0.2)
    gu = torch.stack([g.reshape(I // 16, 16, K), u.reshape(I // 16, 16, K)], 1).reshape(2 * I, K).contiguous()
    gg, uu = a.float() @ g.float().T, a.float() @ u.float().T
    ref = gg / (1 + torch.exp(-gg)) * uu
    out = torch.full((M + 1, I), 7.0, dtype=torch.bfloat16, device=DEV)
    fast().gemm_tc(a, gu, out[:M], fast().EPI_SWIGLU_BF16, tile_n)
    sync_check()
    assert float((out[:M].float() - ref).abs().max()) < 1e-2 * max(1.0, float(ref.abs().max()))
    assert bool((out[M] == 7.0).all())


@pytest.mark.parametrize("M,Hq,Hkv,K,ps,write", [(300, 5, 2, 256, 16, True), (65, 3, 1, 72, 8, True), (2048, 32, 8, 2048, 16, True),
                                               (130, 4, 4, 128, 32, False)])
def test_gemm_tc_rotation_and_cache_write_in_the_epilogue(M, Hq, Hkv, K, ps, write):
    """The q/k/v projection with the rotation and the page writes in its epilogue against the same
    product written out in fp32 and rotated by the kernel of its own: the same bits in q and in
    the pages, pages of rows that are not stored (slot -1) and of other tokens untouched."""
    from hipinfer_b200.kernels import ops

    D = 64
    N = (Hq + 2 * Hkv) * D
    a, w = rnd(M, K, seed=61), ops.Weight(rnd(N, K, seed=62, scale=0.1))
    g = torch.Generator().manual_seed(63)
    n_pos = 4096
    inv_freq = (10000.0 ** (-torch.arange(0, D, 2, dtype=torch.float64) / D)).float().to(DEV)
    table = ops.rope_table(inv_freq, n_pos)
    positions = torch.randint(0, n_pos, (M,), generator=g, dtype=torch.int32).to(DEV)
    n_pages = -(-M // ps) + 4
    slots = torch.randperm(n_pages * ps, generator=g)[:M].to(torch.int32)
    slots[::7] = -1                                             # rows whose keys and values are not stored
    slot_map = slots.to(DEV) if write else None
    fill = lambda: torch.full((n_pages, Hkv, ps, D), 3.0, dtype=torch.bfloat16, device=DEV)
    kc1, vc1, kc2, vc2 = fill(), fill(), fill(), fill()
    q1 = torch.empty(M, Hq * D, dtype=torch.bfloat16, device=DEV)
    q2 = torch.empty_like(q1)
    assert fast().linear_rope_kv(a, w, positions, slot_map, table, q1, kc1, vc1, Hq, Hkv, D, D, ps)
    qkv = torch.empty(M, N, dtype=torch.float32, device=DEV)
    fast().gemm_tc(a, w.t, qkv, fast().EPI_F32)
    ops.rope_kv_write(qkv, positions, slot_map, table, q2, kc2, vc2, Hq, Hkv, D, D, ps)
    sync_check()
    assert torch.equal(q1, q2)
    assert torch.equal(kc1, kc2) and torch.equal(vc1, vc2)
    if write:
        assert float((kc1 != 3.0).float().mean()) > 0.5          # most of the pages were written
    else:
        assert bool((kc1 == 3.0).all()) and bool((vc1 == 3.0).all())


def test_gemm_tc_row_does_not_depend_on_batch():
    """The same row gives the same bits alone, in a small batch and deep inside a large one."""
    a, w = rnd(300, 256, seed=7), rnd(384, 256, seed=8, scale=0.1)
    full = torch.empty(300, 384, dtype=torch.float32, device=DEV)
    fast().gemm_tc(a, w, full, fast().EPI_F32)
    for r in (0, 127, 128, 299):
        one = torch.empty(1, 384, dtype=torch.float32, device=DEV)
        fast().gemm_tc(a[r:r + 1].contiguous(), w, one, fast().EPI_F32)
        sync_check()
        assert torch.equal(one[0], full[r])


def test_gemm_tc_strided_views():
    """Row strides larger than the width (views into wider buffers)."""
    big_a, big_w = rnd(40, 200, seed=9), rnd(96, 264, seed=10, scale=0.1)
    a, w = big_a[:, 8:136], big_w[:, 16:144]
    out_big = torch.zeros(40, 160, dtype=torch.float32, device=DEV)
    out = out_big[:, 32:128]
    fast().gemm_tc(a, w, out, fast().EPI_F32)
    sync_check()
    ref = a.float() @ w.float().T
    assert float((out - ref).abs().max()) < 1e-3
    assert bool((out_big[:, :32] == 0).all()) and bool((out_big[:, 128:] == 0).all())


# ------------------------------------------------------------------------------------------
# the weight-streaming kernel for small batches
# ------------------------------------------------------------------------------------------
IMPLS = ["stream"]


def small(impl):
    return getattr(fast(), "gemm_" + impl)


@pytest.mark.parametrize("impl", IMPLS)
@pytest.mark.parametrize("M", [1, 3, 8, 9, 16, 31, 64])
@pytest.mark.parametrize("N,K", [(128, 128), (96, 72), (300, 200), (1000, 320), (704, 2048), (256, 4104)])
def test_gemm_small(M, N, K, impl):
    a, w = rnd(M, K, seed=11), rnd(N, K, seed=12, scale=0.1)
    ref = a.float().double() @ w.float().double().T
    tol = 2e-5 * max(1.0, float(ref.abs().max())) * (K ** 0.5)
    for _ in range(2):                    # twice: the counters must have been left at zero
        out = torch.full((M + 1, N), 7.0, dtype=torch.float32, device=DEV)
        small(impl)(a, w, out[:M], fast().EPI_F32)
        sync_check()
        assert float((out[:M].double() - ref).abs().max()) < tol
        assert bool((out[M] == 7.0).all()), "wrote past the last row"
    acc = rnd(M, N, seed=13, dtype=torch.float32)
    want = acc.double() + ref
    small(impl)(a, w, acc, fast().EPI_ADD_F32)
    assert float((acc.double() - want).abs().max()) < tol
    ob = torch.empty(M, N, dtype=torch.bfloat16, device=DEV)
    small(impl)(a, w, ob, fast().EPI_BF16)
    assert float((ob.double() - ref).abs().max()) < 1e-2 * max(1.0, float(ref.abs().max()))


@pytest.mark.parametrize("impl", IMPLS)
@pytest.mark.parametrize("M,I,K", [(1, 16, 64), (5, 176, 96), (17, 320, 136), (64, 1024, 2048)])
def test_gemm_small_swiglu(M, I, K, impl):
    a = rnd(M, K, seed=14)
    g, u = rnd(I, K, seed=15, scale=0.2), rnd(I, K, seed=16, scale=0.2)
    gu = torch.stack([g.reshape(I // 16, 16, K), u.reshape(I // 16, 16, K)], 1).reshape(2 * I, K).contiguous()
    gg, uu = a.float() @ g.float().T, a.float() @ u.float().T
    ref = gg / (1 + torch.exp(-gg)) * uu
    out = torch.full((M + 1, I), 7.0, dtype=torch.bfloat16, device=DEV)
    small(impl)(a, gu, out[:M], fast().EPI_SWIGLU_BF16)
    assert float((out[:M].float() - ref).abs().max()) < 1e-2 * max(1.0, float(ref.abs().max()))
    assert bool((out[M] == 7.0).all())


@pytest.mark.parametrize("impl", IMPLS)
def test_gemm_small_row_does_not_depend_on_batch(impl):
    """A token's result is bit-identical alone, among 8 and among 64 (the K split depends on the weight only)."""
    a, w = rnd(64, 2048, seed=17), rnd(384, 2048, seed=18, scale=0.1)
    full = torch.empty(64, 384, dtype=torch.float32, device=DEV)
    small(impl)(a, w, full, fast().EPI_F32)
    for rows in ([0], [5, 63], list(range(3, 12)), list(range(20, 50))):
        sub = torch.empty(len(rows), 384, dtype=torch.float32, device=DEV)
        small(impl)(a[rows].contiguous(), w, sub, fast().EPI_F32)
        assert torch.equal(sub, full[rows])


@pytest.mark.parametrize("impl", IMPLS)
def test_small_and_tile_kernels_agree_to_rounding(impl):
    a, w = rnd(64, 1024, seed=19), rnd(512, 1024, seed=20, scale=0.1)
    x, y = torch.empty(64, 512, device=DEV), torch.empty(64, 512, device=DEV)
    small(impl)(a, w, x, fast().EPI_F32)
    fast().gemm_tc(a, w, y, fast().EPI_F32)
    sync_check()
    assert float((x - y).abs().max()) < 1e-4 * float(y.abs().max())


# ------------------------------------------------------------------------------------------
# attention over the paged bf16 cache
# ------------------------------------------------------------------------------------------
import math

import plain_llama as plain
from test_gpu_kernels_plain import _paged_setup


@pytest.mark.parametrize("Hq,Hkv,D,ps,window", [(8, 2, 64, 16, 0), (3, 1, 128, 8, 0), (10, 2, 128, 16, 0), (8, 8, 64, 32, 0),
                                                (8, 1, 64, 16, 0), (6, 2, 64, 16, 40), (4, 2, 64, 16, 300), (7, 1, 64, 16, 0),
                                                (4, 1, 128, 32, 0), (4, 2, 128, 64, 0), (8, 1, 128, 16, 0)])
def test_attention_decode(Hq, Hkv, D, ps, window):
    lens = [700, 37, 1, 300]
    kc, vc, bt, ks, vs = _paged_setup(lens, Hkv, D, ps, torch.bfloat16, 21)
    rows = [(0, 699), (1, 30), (1, 31), (1, 36), (2, 0), (3, 255), (3, 256), (3, 299), (0, 511), (0, 512)]
    T = len(rows)
    q = rnd(T, Hq * D, seed=22)
    qf = q.float().cpu().reshape(T, Hq, D)
    out = torch.empty(T, Hq * D, dtype=torch.bfloat16, device=DEV)
    rr = torch.tensor([r for r, _ in rows], dtype=torch.int32, device=DEV)
    pos = torch.tensor([p for _, p in rows], dtype=torch.int32, device=DEV)
    fast().attention_decode(q, kc, vc, bt, rr, pos, out, Hq, Hkv, D, ps, window, 1.0 / math.sqrt(D), max(p for _, p in rows))
    # the same with the keys of earlier steps asked for early (requests 1 and 3 have several rows:
    # their new keys start at the first row's position): bit-identical
    early = torch.full_like(out, 3.0)
    ctx = torch.tensor([511, 30, 0, 255], dtype=torch.int32, device=DEV)
    torch.cuda.synchronize()
    for _ in range(2):      # twice: the counters are left at zero
        fast().attention_decode(q, kc, vc, bt, rr, pos, early, Hq, Hkv, D, ps, window, 1.0 / math.sqrt(D),
                                max(p for _, p in rows), ctx_len=ctx)
        assert torch.equal(early, out)
        early.fill_(3.0)
    got = out.float().cpu().reshape(T, Hq, D)
    for t, (r, p) in enumerate(rows):
        ref = plain.attention_scores_softmax_values(qf[t:t + 1], ks[r][:p + 1], vs[r][:p + 1], [p], list(range(p + 1)),
                                                    window or None)
        torch.testing.assert_close(got[t:t + 1], ref, rtol=1e-2, atol=1e-2, msg=lambda m: f"row {t} {rows[t]}: {m}")


@pytest.mark.parametrize("D", [64, 128])
def test_attention_decode_long_context_many_chunks(D):
    """4,500 keys: 18 chunks of 256, more than the merge keeps in registers at once (its other path)."""
    Hq, Hkv, ps = 4, 1, 16
    kc, vc, bt, ks, vs = _paged_setup([4500, 300], Hkv, D, ps, torch.bfloat16, 25)
    rows = [(0, 4499), (1, 299), (0, 4096), (0, 4095)]
    q = rnd(len(rows), Hq * D, seed=26)
    qf = q.float().cpu().reshape(len(rows), Hq, D)
    out = torch.empty(len(rows), Hq * D, dtype=torch.bfloat16, device=DEV)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    fast().attention_decode(q, kc, vc, bt, i32([r for r, _ in rows]), i32([p for _, p in rows]), out, Hq, Hkv, D, ps, 0,
                            1 / math.sqrt(D), 4499, ctx_len=i32([4095, 299]))
    sync_check()
    got = out.float().cpu().reshape(len(rows), Hq, D)
    for t, (r, p) in enumerate(rows):
        ref = plain.attention_scores_softmax_values(qf[t:t + 1], ks[r][:p + 1], vs[r][:p + 1], [p], list(range(p + 1)))
        torch.testing.assert_close(got[t:t + 1], ref, rtol=1e-2, atol=1e-2, msg=lambda m: f"row {t} {rows[t]}: {m}")


@pytest.mark.parametrize("D", [64, 128])
def test_attention_decode_few_and_many_rows_give_the_same_bits(D):
    """With few rows every block has an SM of its own and takes all its keys at once; with many a warp
    asks for its keys pass by pass: the passes are the same, so a row's result is bit-identical."""
    Hq, Hkv, ps = 32, 8, 16
    lens = [1500, 700, 2300]
    kc, vc, bt, ks, vs = _paged_setup(lens, Hkv, D, ps, torch.bfloat16, 71)
    rows = [(r, p) for r, n in enumerate(lens) for p in range(n - 14, n)]          # 42 rows: 42 * 8 * 5 blocks
    q = rnd(len(rows), Hq * D, seed=72)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    scale = 1 / math.sqrt(D)
    many = torch.empty(len(rows), Hq * D, dtype=torch.bfloat16, device=DEV)
    fast().attention_decode(q, kc, vc, bt, i32([r for r, _ in rows]), i32([p for _, p in rows]), many, Hq, Hkv, D, ps, 0, scale,
                            max(lens) - 1)
    for pick in ([0], [13, 14], [41]):
        few = torch.empty(len(pick), Hq * D, dtype=torch.bfloat16, device=DEV)
        fast().attention_decode(q[pick].contiguous(), kc, vc, bt, i32([rows[i][0] for i in pick]), i32([rows[i][1] for i in pick]),
                                few, Hq, Hkv, D, ps, 0, scale, max(lens) - 1)
        sync_check()
        assert torch.equal(few, many[pick])
    t = 41
    r, p = rows[t]
    ref = plain.attention_scores_softmax_values(q[t:t + 1].float().cpu().reshape(1, Hq, D), ks[r][:p + 1], vs[r][:p + 1], [p],
                                                list(range(p + 1)))
    torch.testing.assert_close(many[t:t + 1].float().cpu().reshape(1, Hq, D), ref, rtol=1e-2, atol=1e-2)


def test_attention_decode_rows_that_are_requests():
    """A decode-only step: row t is request t, which the kernel then does not look up: the same bits."""
    Hq, Hkv, D, ps = 8, 2, 64, 16
    lens = [700, 37, 1, 300, 257]
    kc, vc, bt, ks, vs = _paged_setup(lens, Hkv, D, ps, torch.bfloat16, 27)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    q = rnd(len(lens), Hq * D, seed=28)
    pos, rr = i32([n - 1 for n in lens]), i32(list(range(len(lens))))
    a, b = (torch.empty(len(lens), Hq * D, dtype=torch.bfloat16, device=DEV) for _ in range(2))
    fast().attention_decode(q, kc, vc, bt, rr, pos, a, Hq, Hkv, D, ps, 0, 1 / math.sqrt(D), max(lens) - 1, ctx_len=pos)
    fast().attention_decode(q, kc, vc, bt, None, pos, b, Hq, Hkv, D, ps, 0, 1 / math.sqrt(D), max(lens) - 1, ctx_len=pos)
    sync_check()
    assert torch.equal(a, b)


def test_attention_decode_far_key_stands_out():
    Hq, Hkv, D, ps = 4, 1, 64, 16
    kc, vc, bt, ks, vs = _paged_setup([900], Hkv, D, ps, torch.bfloat16, 23)
    q = rnd(1, Hq * D, seed=24)
    qf = q.float().cpu().reshape(1, Hq, D)
    far = 5
    page, off = int(bt[0, far // ps]), far % ps
    kc[page, 0, off] = (qf[0, 0] * 4.0).to(torch.bfloat16).to(DEV)
    ks[0][far, 0] = kc[page, 0, off].float().cpu()
    out = torch.empty(1, Hq * D, dtype=torch.bfloat16, device=DEV)
    fast().attention_decode(q, kc, vc, bt, torch.zeros(1, dtype=torch.int32, device=DEV),
                            torch.tensor([899], dtype=torch.int32, device=DEV), out, Hq, Hkv, D, ps, 0, 1 / math.sqrt(D), 899)
    ref = plain.attention_scores_softmax_values(qf, ks[0], vs[0], [899], list(range(900)))
    torch.testing.assert_close(out.float().cpu().reshape(1, Hq, D), ref, rtol=1e-2, atol=1e-2)
    assert float((out.float().cpu().reshape(Hq, D)[0] - vs[0][far, 0]).abs().max()) < 0.05


FLASH = ["flash_prefill", "flash_prefill_tc"]


@pytest.mark.parametrize("impl", FLASH)
@pytest.mark.parametrize("Hq,Hkv,D,ps,window", [(8, 2, 64, 16, 0), (3, 1, 128, 16, 0), (4, 4, 64, 8, 0), (6, 2, 64, 16, 100),
                                                (2, 1, 128, 32, 0), (5, 1, 64, 32, 0)])
def test_flash_prefill(Hq, Hkv, D, ps, window, impl):
    if impl == "flash_prefill_tc" and not fast().flash_prefill_tc_supported(Hq, Hkv, D, ps):
        pytest.skip("the tcgen05 kernel takes head_dim 64")
    """Portions of several requests in one launch: a whole prompt from position 0 with a ragged
    last tile, a portion in the middle of a sequence that starts inside a page and inside a key
    tile, a long portion behind a long context, and a short portion that must be left alone."""
    ctx = [0, 83, 400, 50]
    qn = [150, 77, 130, 5]
    lens = [c + n for c, n in zip(ctx, qn)]
    kc, vc, bt, ks, vs = _paged_setup(lens, Hkv, D, ps, torch.bfloat16, 31)
    T = sum(qn)
    q = rnd(T, Hq * D, seed=32)
    qf = q.float().cpu().reshape(T, Hq, D)
    out = torch.full((T, Hq * D), 7.0, dtype=torch.bfloat16, device=DEV)
    starts = [sum(qn[:i]) for i in range(4)]
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    getattr(fast(), impl)(q, kc, vc, bt, i32(starts), i32(qn), i32(ctx), out, max(qn), Hq, Hkv, D, ps, window,
                          1.0 / math.sqrt(D), min_rows=16)
    sync_check()
    got = out.float().cpu().reshape(T, Hq, D)
    for r in range(3):
        pos = list(range(ctx[r], ctx[r] + qn[r]))
        ref = plain.attention_scores_softmax_values(qf[starts[r]:starts[r] + qn[r]], ks[r], vs[r], pos, list(range(lens[r])),
                                                    window or None)
        torch.testing.assert_close(got[starts[r]:starts[r] + qn[r]], ref, rtol=2e-2, atol=2e-2,
                                   msg=lambda m: f"request {r}: {m}")
    assert bool((got[starts[3]:] == 7.0).all()), "the short portion was touched"


@pytest.mark.parametrize("impl", FLASH)
def test_flash_prefill_far_key_and_cutting(impl):
    """A far key made to stand out comes through; the same rows cut into two portions give the same bits."""
    Hq, Hkv, D, ps = 4, 2, 64, 16
    n = 600
    kc, vc, bt, ks, vs = _paged_setup([n], Hkv, D, ps, torch.bfloat16, 33)
    q = rnd(n, Hq * D, seed=34)
    qf = q.float().cpu().reshape(n, Hq, D)
    far, row = 7, 555
    page, off = int(bt[0, far // ps]), far % ps
    kc[page, 0, off] = (qf[row, 0] * 4.0).to(torch.bfloat16).to(DEV)
    ks[0][far, 0] = kc[page, 0, off].float().cpu()
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    whole = torch.empty(n, Hq * D, dtype=torch.bfloat16, device=DEV)
    flash = getattr(fast(), impl)
    flash(q, kc, vc, bt, i32([0]), i32([n]), i32([0]), whole, n, Hq, Hkv, D, ps, 0, 1 / math.sqrt(D))
    sync_check()
    ref = plain.attention_scores_softmax_values(qf, ks[0], vs[0], list(range(n)), list(range(n)))
    torch.testing.assert_close(whole.float().cpu().reshape(n, Hq, D), ref, rtol=2e-2, atol=2e-2)
    assert float((whole.float().cpu().reshape(n, Hq, D)[row, 0] - vs[0][far, 0]).abs().max()) < 0.05
    cut = 333
    tail = torch.empty(n - cut, Hq * D, dtype=torch.bfloat16, device=DEV)
    flash(q[cut:].contiguous(), kc, vc, bt, i32([0]), i32([n - cut]), i32([cut]), tail, n - cut, Hq, Hkv, D, ps, 0,
          1 / math.sqrt(D))
    sync_check()
    assert torch.equal(tail, whole[cut:])


@pytest.mark.parametrize("impl", FLASH)
@pytest.mark.parametrize("D", [64, 128])
def test_flash_prefill_running_maximum(impl, D):
    """Scores that climb along the keys, so that the running maximum of a row keeps rising: by about 5
    binary orders a key tile (a kernel that follows the maximum lazily lets several tiles pass before
    it rescales the output), by about 20 (rescaled at every tile), falling (the first tile holds the
    maximum and later tiles add almost nothing), and flat at a large magnitude."""
    Hq, Hkv, ps, n = 4, 2, 16, 1100
    if impl == "flash_prefill_tc" and not fast().flash_prefill_tc_supported(Hq, Hkv, D, ps):
        pytest.skip("not a size of the tcgen05 kernel")
    g = torch.Generator().manual_seed(51)
    u = (torch.randint(0, 2, (D,), generator=g).float() * 2 - 1)            # +-1: |u|^2 = D
    pos = torch.arange(n, dtype=torch.float32)
    slope = 5.0 / 1.4427 / 128 / math.sqrt(D)                                 # q.k / sqrt(D) grows by 5 / log2(e) in 128 keys
    k = torch.randn(n, Hkv, D, generator=g) * 0.05
    k[:, 0] += u[None] * (pos * slope)[:, None]                              # kv head 0: climbing
    k[:, 1] += u[None] * ((n - pos) * slope)[:, None]                        # kv head 1: falling
    k = k.to(torch.bfloat16)
    v = torch.randn(n, Hkv, D, generator=g).to(torch.bfloat16)
    q = torch.randn(n, Hq, D, generator=g) * 0.05
    q[:, 0] += u      # slow climb
    q[:, 1] += 4 * u  # fast climb
    q[:, 2] += u      # falling
    q[:, 3] += 0      # flat and small; made large below
    q[:, 3] *= 40
    q = q.to(torch.bfloat16)
    n_pages = -(-n // ps)
    kc = torch.zeros(n_pages, Hkv, ps, D, dtype=torch.bfloat16)
    vc = torch.zeros_like(kc)
    for lp in range(n_pages):
        m = min(ps, n - lp * ps)
        kc[lp, :, :m] = k[lp * ps:lp * ps + m].transpose(0, 1)
        vc[lp, :, :m] = v[lp * ps:lp * ps + m].transpose(0, 1)
    bt = torch.arange(n_pages, dtype=torch.int32).view(1, -1).to(DEV)
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=DEV)
    out = torch.empty(n, Hq * D, dtype=torch.bfloat16, device=DEV)
    getattr(fast(), impl)(q.reshape(n, Hq * D).to(DEV), kc.to(DEV), vc.to(DEV), bt, i32([0]), i32([n]), i32([0]), out, n,
                          Hq, Hkv, D, ps, 0, 1 / math.sqrt(D))
    sync_check()
    ref = plain.attention_scores_softmax_values(q.float(), k.float(), v.float(), list(range(n)), list(range(n)))
    got = out.float().cpu().reshape(n, Hq, D)
    for h in range(Hq):
        torch.testing.assert_close(got[:, h], ref[:, h], rtol=2e-2, atol=2e-2, msg=lambda m: f"head {h}: {m}")


# ------------------------------------------------------------------------------------------
# small products left as K slices, and the kernels that consume them
# ------------------------------------------------------------------------------------------
@pytest.mark.parametrize("M,H,K", [(1, 2048, 2048), (8, 2048, 8192), (13, 520, 352), (40, 3072, 1024), (64, 4096, 256)])
def test_slices_added_by_the_norm(M, H, K):
    """x += a w^T and RMSNorm(x) with the slices added by the norm kernel: x bit-identical to the
    product finishing itself, the norm equal to the plain norm after it up to the rounding of its
    sum of squares (another order) and of the result to bfloat16; also on gathered rows, where x stays."""
    from hipinfer_b200.kernels import ops

    a, w = rnd(M, K, seed=41), ops.Weight(rnd(H, K, seed=42, scale=0.05))
    x0 = rnd(M, H, seed=43, scale=2.0, dtype=torch.float32)
    nw = (1 + rnd(H, seed=44, dtype=torch.float32) * 0.1).to(torch.bfloat16)
    x_ref = x0.clone()
    ops.linear(a, w, x_ref, accumulate=True)
    y_ref = ops.rmsnorm(x_ref, nw, 1e-5, torch.empty(M, H, dtype=torch.bfloat16, device=DEV))
    want = x0.float().cpu() + a.float().cpu() @ w.t.float().cpu().T
    assert float((x_ref.cpu() - want).abs().max()) < 1e-3 * float(want.abs().max())
    x = x0.clone()
    pend = ops.linear_deferred(a, w, x, accumulate=True)
    assert pend is not None and torch.equal(x, x0)          # nothing added yet
    y = ops.rmsnorm(x, nw, 1e-5, torch.full((M, H), 3.0, dtype=torch.bfloat16, device=DEV), pending=pend)
    sync_check()
    assert torch.equal(x, x_ref)
    ulp = lambda got, ref: float(((got.float() - ref.float()).abs() / ref.float().abs().clamp_min(1e-3)).max())
    assert ulp(y, y_ref) <= 2.0 ** -7 and float((y != y_ref).float().mean()) < 0.01
    rows = torch.tensor([M - 1, 0, M - 1], dtype=torch.int32, device=DEV)
    x = x0.clone()
    pend = ops.linear_deferred(a, w, x, accumulate=True)
    y2 = ops.rmsnorm(x, nw, 1e-5, torch.empty(3, H, dtype=torch.bfloat16, device=DEV), rows=rows, pending=pend)
    assert torch.equal(y2, y[[M - 1, 0, M - 1]]) and torch.equal(x, x0)
    # finished by hand, and the guard against a product in between
    x = x0.clone()
    ops.linear_deferred(a, w, x, accumulate=True).finish()
    assert torch.equal(x, x_ref)
    pend = ops.linear_deferred(a, w, x, accumulate=True)
    ops.linear(a, w, torch.empty(M, H, device=DEV))
    with pytest.raises(RuntimeError, match="overwritten"):
        pend.finish()


@pytest.mark.parametrize("M,Hq,Hkv,D,K", [(1, 32, 8, 64, 2048), (8, 32, 8, 64, 2048), (16, 8, 2, 64, 256), (5, 4, 2, 128, 512),
                                          (37, 3, 1, 72, 72)])
def test_slices_added_by_the_rotation(M, Hq, Hkv, D, K):
    """q/k/v product, rotation and cache write with the slices added by the rotation kernel:
    bit-identical to the three steps one after the other."""
    from hipinfer_b200.kernels import ops
    from hipinfer_b200.parts.rotary import rope_inv_freq

    ps, n_pages = 16, 6
    N = (Hq + 2 * Hkv) * D
    xn = rnd(M, K, seed=51)
    w = ops.Weight(rnd(N, K, seed=53, scale=0.05))
    table = ops.rope_table(rope_inv_freq(D, 500000.0).to(DEV), 128)
    g = torch.Generator().manual_seed(54)
    pos = torch.randint(0, 128, (M,), generator=g).to(torch.int32).to(DEV)
    slots = torch.randperm(ps * n_pages, generator=g)[:M].to(torch.int32).to(DEV)
    qkv = torch.empty(M, N, dtype=torch.float32, device=DEV)
    ops.linear(xn, w, qkv)
    q_ref = torch.empty(M, Hq * D, dtype=torch.bfloat16, device=DEV)
    kc_ref = torch.full((n_pages, Hkv, ps, D), 9.0, dtype=torch.bfloat16, device=DEV)
    vc_ref = kc_ref.clone()
    ops.rope_kv_write(qkv, pos, slots, table, q_ref, kc_ref, vc_ref, Hq, Hkv, D, D, ps)
    q = torch.empty_like(q_ref)
    kc, vc = torch.full_like(kc_ref, 9.0), torch.full_like(vc_ref, 9.0)
    pend = ops.linear_deferred(xn, w, qkv)
    assert pend is not None
    ops.rope_kv_write(qkv, pos, slots, table, q, kc, vc, Hq, Hkv, D, D, ps, pending=pend)
    sync_check()
    assert torch.equal(q, q_ref) and torch.equal(kc, kc_ref) and torch.equal(vc, vc_ref)
    kc2 = torch.full_like(kc_ref, 9.0)                      # without a slot map nothing is stored
    ops.rope_kv_write(qkv, pos, None, table, q, kc2, kc2, Hq, Hkv, D, D, ps, pending=ops.linear_deferred(xn, w, qkv))
    torch.cuda.synchronize()
    assert bool((kc2 == 9.0).all()) and torch.equal(q, q_ref)


# ------------------------------------------------------------------------------------------
# the kernels for a few token rows: whole-K stripes, the norm in the prologue, the layer's arithmetic in the epilogue
# ------------------------------------------------------------------------------------------
def _rms(x, w, eps):
    """RMSNorm in float64 from float32 rows, rounded once to bfloat16 (what the product then reads)."""
    xd = x.double()
    return (w.double() * (xd * torch.rsqrt((xd * xd).mean(-1, keepdim=True) + eps))).float().bfloat16()


@pytest.mark.parametrize("M", [1, 3, 8, 9, 16])
@pytest.mark.parametrize("N,K", [(128, 128), (96, 96), (300, 224), (2048, 8192), (704, 2048), (40, 1056)])
def test_rows_add(M, N, K):
    """out += act W^T finished in one kernel, twice in a row, nothing written beyond the last row or column."""
    a, w = rnd(M, K, seed=71), rnd(N, K, seed=72, scale=0.1)
    ref = a.float().double() @ w.float().double().T
    tol = 2e-5 * max(1.0, float(ref.abs().max())) * (K ** 0.5)
    for _ in range(2):
        base = rnd(M + 1, N + 3, seed=73, dtype=torch.float32)
        out = base.clone()
        assert fast().rows_add(a, w, out[:M, :N])
        sync_check()
        assert float((out[:M, :N].double() - (base[:M, :N].double() + ref)).abs().max()) < tol
        assert torch.equal(out[M], base[M]) and torch.equal(out[:, N:], base[:, N:])


@pytest.mark.parametrize("M,I,K", [(1, 16, 64), (5, 176, 96), (8, 320, 160), (16, 1024, 2048), (7, 8192, 3072), (12, 48, 4096)])
def test_rows_norm_swiglu(M, I, K):
    x = rnd(M, K, seed=74, dtype=torch.float32, scale=3.0)
    nw = (1 + 0.2 * torch.randn(K, generator=torch.Generator().manual_seed(75))).bfloat16().to(DEV)
    g, u = rnd(I, K, seed=76, scale=0.2), rnd(I, K, seed=77, scale=0.2)
    gu = torch.stack([g.reshape(I // 16, 16, K), u.reshape(I // 16, 16, K)], 1).reshape(2 * I, K).contiguous()
    xn = _rms(x, nw, 1e-5).float()
    gg, uu = xn @ g.float().T, xn @ u.float().T
    ref = gg / (1 + torch.exp(-gg)) * uu
    out = torch.full((M + 1, I), 7.0, dtype=torch.bfloat16, device=DEV)
    assert fast().rows_norm_swiglu(x, nw, 1e-5, gu, out[:M], 16)
    sync_check()
    assert float((out[:M].float() - ref).abs().max()) < 1.5e-2 * max(1.0, float(ref.abs().max()))
    assert bool((out[M] == 7.0).all())


@pytest.mark.parametrize("M,Hq,Hkv,D,K,ps,write", [(1, 32, 8, 64, 2048, 16, True), (8, 32, 8, 64, 2048, 16, True), (16, 8, 2, 64, 256, 8, True),
                                                   (5, 4, 2, 128, 512, 16, True), (3, 3, 1, 32, 96, 16, True), (9, 4, 2, 16, 64, 16, True),
                                                   (6, 24, 8, 128, 3072, 16, True), (4, 4, 4, 64, 128, 32, False)])
def test_rows_norm_qkv_rope(M, Hq, Hkv, D, K, ps, write):
    """Norm, projection, rotation and page writes as one kernel against the same steps in float32/float64: q and
    the pages within bfloat16 rounding of the plain result, pages of other tokens and of rows that are not stored untouched."""
    from hipinfer_b200.kernels import ops

    N = (Hq + 2 * Hkv) * D
    x = rnd(M, K, seed=81, dtype=torch.float32, scale=2.0)
    nw = (1 + 0.2 * torch.randn(K, generator=torch.Generator().manual_seed(82))).bfloat16().to(DEV)
    w = rnd(N, K, seed=83, scale=0.1)
    g = torch.Generator().manual_seed(84)
    n_pos = 4096
    inv_freq = (10000.0 ** (-torch.arange(0, D, 2, dtype=torch.float64) / D)).float().to(DEV)
    table = ops.rope_table(inv_freq, n_pos)
    positions = torch.randint(0, n_pos, (M,), generator=g, dtype=torch.int32).to(DEV)
    n_pages = -(-M // ps) + 4
    slots = torch.randperm(n_pages * ps, generator=g)[:M].to(torch.int32)
    if M > 2:
        slots[2] = -1                                           # a row whose key and value are not stored
    slot_map = slots.to(DEV) if write else None
    kc = torch.full((n_pages, Hkv, ps, D), 3.0, dtype=torch.bfloat16, device=DEV)
    vc = kc.clone()
    q = torch.full((M + 1, Hq * D), 7.0, dtype=torch.bfloat16, device=DEV)
    assert fast().rows_norm_qkv_rope(x, nw, 1e-5, w, positions, slot_map, table, q[:M], kc, vc, Hq, Hkv, D, D, ps)
    sync_check()
    # plain: norm (rounded once), product in float64, rotation of the pairs (j, j + D/2)
    qkv = (_rms(x, nw, 1e-5).double() @ w.double().T)
    cs = table[positions.long()].double()                       # [M, D/2, 2]
    cos, sin = cs[..., 0][:, None, :], cs[..., 1][:, None, :]

    def rot(t):
        t1, t2 = t[..., :D // 2], t[..., D // 2:]
        return torch.cat([t1 * cos - t2 * sin, t2 * cos + t1 * sin], -1)

    q_ref = rot(qkv[:, :Hq * D].reshape(M, Hq, D)).reshape(M, Hq * D)
    k_ref = rot(qkv[:, Hq * D:(Hq + Hkv) * D].reshape(M, Hkv, D))
    v_ref = qkv[:, (Hq + Hkv) * D:].reshape(M, Hkv, D)
    tol = 1.2e-2 * max(1.0, float(qkv.abs().max()))
    assert float((q[:M].double() - q_ref).abs().max()) < tol
    assert bool((q[M] == 7.0).all())
    kc_ref = torch.full_like(kc, 3.0).double()
    vc_ref = kc_ref.clone()
    if write:
        for m in range(M):
            s = int(slots[m])
            if s >= 0:
                kc_ref[s // ps, :, s % ps] = k_ref[m]
                vc_ref[s // ps, :, s % ps] = v_ref[m]
    untouched = kc_ref == 3.0
    assert float((kc.double() - kc_ref).abs().max()) < tol and float((vc.double() - vc_ref).abs().max()) < tol
    assert bool((kc[untouched] == 3.0).all()) and bool((vc[vc_ref == 3.0] == 3.0).all())


def test_rows_kernels_do_not_depend_on_the_batch():
    """A token's result is bit-identical alone, among 8 and among 16 rows (its column of the MMA is its own)."""
    from hipinfer_b200.kernels import ops

    K, I, Hq, Hkv, D, ps = 2048, 512, 8, 2, 64, 16
    x = rnd(16, K, seed=91, dtype=torch.float32, scale=2.0)
    nw = torch.ones(K, dtype=torch.bfloat16, device=DEV)
    gu, wo, wqkv = rnd(2 * I, K, seed=92, scale=0.1), rnd(384, K, seed=93, scale=0.1), rnd((Hq + 2 * Hkv) * D, K, seed=94, scale=0.1)
    act = rnd(16, K, seed=95)
    table = ops.rope_table((10000.0 ** (-torch.arange(0, D, 2, dtype=torch.float64) / D)).float().to(DEV), 512)
    pos = torch.arange(100, 116, dtype=torch.int32, device=DEV)

    def run(rows):
        r = torch.tensor(rows, device=DEV)
        n = len(rows)
        o1 = torch.empty(n, I, dtype=torch.bfloat16, device=DEV)
        assert fast().rows_norm_swiglu(x[r].contiguous(), nw, 1e-5, gu, o1, 16)
        o2 = torch.zeros(n, 384, dtype=torch.float32, device=DEV)
        assert fast().rows_add(act[r].contiguous(), wo, o2)
        q = torch.empty(n, Hq * D, dtype=torch.bfloat16, device=DEV)
        assert fast().rows_norm_qkv_rope(x[r].contiguous(), nw, 1e-5, wqkv, pos[r].contiguous(), None, table, q, None, None,
                                         Hq, Hkv, D, D, ps)
        sync_check()
        return o1, o2, q

    full = run(list(range(16)))
    for rows in ([0], [5, 15], list(range(3, 11)), list(range(2, 14))):
        for got, want in zip(run(rows), full):
            assert torch.equal(got, want[rows])


def test_rows_kernels_refuse_what_they_do_not_take():
    x = rnd(17, 256, seed=96, dtype=torch.float32)
    nw = torch.ones(256, dtype=torch.bfloat16, device=DEV)
    w = rnd(64, 256, seed=97)
    out = torch.zeros(17, 32, dtype=torch.bfloat16, device=DEV)
    assert not fast().rows_norm_swiglu(x, nw, 1e-5, w, out, 16)                    # 17 rows
    assert not fast().rows_norm_swiglu(x[:4], nw, 1e-5, w.float(), out[:4], 16)    # weights stored in 32-bit
    assert not fast().rows_add(rnd(4, 200, seed=98), rnd(64, 200, seed=99), torch.zeros(4, 64, device=DEV))   # K no multiple of 32
    assert not fast().rows_norm_swiglu(rnd(4, 65536, seed=1, dtype=torch.float32), torch.ones(65536, dtype=torch.bfloat16, device=DEV),
                                       1e-5, rnd(32, 65536, seed=2), out[:4, :16], 16)   # rows too wide for shared memory


@pytest.mark.parametrize("M,H,I,Hq,Hkv,D", [(8, 2048, 1024, 8, 2, 64), (1, 256, 96, 4, 2, 32), (5, 3072, 512, 6, 2, 128), (13, 512, 160, 4, 4, 16)])
def test_rows_add_prepares_the_next_norm(M, H, I, Hq, Hkv, D):
    """The residual add that also leaves x * (next norm's weight) in bf16 and the pieces of the rows' sums of squares,
    and the two products that take those in place of the residual rows (1 / RMS in their epilogue): against the plain
    statement (norm rounded once, products in float64), and x itself the same bits as without the preparation."""
    from hipinfer_b200.kernels import ops

    act, wd = rnd(M, I, seed=101), rnd(H, I, seed=102, scale=0.1)
    x0 = rnd(M, H, seed=103, dtype=torch.float32, scale=2.0)
    nw = (1 + 0.2 * torch.randn(H, generator=torch.Generator().manual_seed(104))).bfloat16().to(DEV)
    feed = fast().NormFeed(nw, 1e-5, M)
    x1, x2 = x0.clone(), x0.clone()
    assert fast().rows_add(act, wd, x1, feed) and feed.filled
    assert fast().rows_add(act, wd, x2)
    sync_check()
    assert torch.equal(x1, x2)
    assert float((feed.xb.float() - x1 * nw.float()).abs().max()) <= 2 ** -8 * float((x1 * nw.float()).abs().max())
    ssq = feed.ssq.sum(0)[:M].double()
    assert float((ssq - (x1.double() ** 2).sum(-1)).abs().max()) < 1e-4 * float(ssq.max())
    xn = _rms(x1, nw, 1e-5).double()
    # gate/up from the feed
    g, u = rnd(I, H, seed=105, scale=0.2), rnd(I, H, seed=106, scale=0.2)
    gu = torch.stack([g.reshape(I // 16, 16, H), u.reshape(I // 16, 16, H)], 1).reshape(2 * I, H).contiguous()
    gg, uu = xn @ g.double().T, xn @ u.double().T
    ref = gg / (1 + torch.exp(-gg)) * uu
    out = torch.full((M + 1, I), 7.0, dtype=torch.bfloat16, device=DEV)
    assert fast().rows_scaled_swiglu(feed, M, gu, out[:M], 16)
    sync_check()
    assert float((out[:M].double() - ref).abs().max()) < 1.5e-2 * max(1.0, float(ref.abs().max()))
    assert bool((out[M] == 7.0).all())
    # q/k/v with rotation from the feed, against the kernel that normalises itself
    N = (Hq + 2 * Hkv) * D
    w = rnd(N, H, seed=107, scale=0.1)
    table = ops.rope_table((10000.0 ** (-torch.arange(0, D, 2, dtype=torch.float64) / D)).float().to(DEV), 512)
    pos = torch.arange(M, dtype=torch.int32, device=DEV) * 7 + 3
    slots = torch.arange(M, dtype=torch.int32, device=DEV) * 3 + 1
    mk = lambda: torch.full((M * 3 // 16 + 2, Hkv, 16, D), 3.0, dtype=torch.bfloat16, device=DEV)
    kc1, vc1, kc2, vc2 = mk(), mk(), mk(), mk()
    q1 = torch.empty(M, Hq * D, dtype=torch.bfloat16, device=DEV)
    q2 = torch.empty_like(q1)
    assert fast().rows_scaled_qkv_rope(feed, M, w, pos, slots, table, q1, kc1, vc1, Hq, Hkv, D, D, 16)
    assert fast().rows_norm_qkv_rope(x1, nw, 1e-5, w, pos, slots, table, q2, kc2, vc2, Hq, Hkv, D, D, 16)
    sync_check()
    scale = max(1.0, float(q2.float().abs().max()))
    for a, b in ((q1, q2), (kc1, kc2), (vc1, vc2)):      # the two round the activations at different places: bf16 rounding apart
        assert float((a.float() - b.float()).abs().max()) < 2e-2 * scale
