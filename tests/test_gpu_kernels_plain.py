"""Each plain kernel alone beside a plain PyTorch float32 statement of the same operation, at
sizes other than the engine's: widths that are no power of two, odd row counts, head sizes in
steps of 16, groups of 1, 3, 5."""
import math

import pytest
import torch

import plain_llama as plain

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
DT = [torch.float32, torch.bfloat16]


def ops():
    from hipinfer_b200.kernels import ops as o
    return o


def rnd(*shape, dtype=torch.float32, seed=0, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(dtype).to(DEV)


@pytest.mark.parametrize("dtype", DT)
def test_embedding(dtype):
    table = rnd(301, 72, dtype=dtype)
    tok = torch.tensor([0, 300, 7, 7, 150], dtype=torch.int32, device=DEV)
    out = torch.empty(5, 72, dtype=torch.float32, device=DEV)
    ops().embedding(table, tok, out)
    assert torch.equal(out, plain.embed(tok.cpu().tolist(), table.float().cpu()).to(DEV))


@pytest.mark.parametrize("wdt", DT)
@pytest.mark.parametrize("odt", DT)
@pytest.mark.parametrize("M,H,eps", [(1, 64, 1e-5), (7, 200, 1e-6), (33, 2048, 1e-5), (3, 3000, 1e-3)])
def test_rmsnorm(wdt, odt, M, H, eps):
    x = rnd(M, H, scale=3.0, seed=1)
    w = (1 + rnd(H, seed=2) * 0.1).to(wdt)
    out = torch.empty(M, H, dtype=odt, device=DEV)
    ops().rmsnorm(x, w, eps, out)
    ref = plain.rmsnorm(x.cpu(), w.float().cpu(), eps)
    tol = 1e-5 if odt == torch.float32 else 1e-2
    torch.testing.assert_close(out.float().cpu(), ref, rtol=tol, atol=tol)
    rows = torch.tensor([M - 1, 0], dtype=torch.int32, device=DEV)
    out2 = torch.empty(2, H, dtype=odt, device=DEV)
    ops().rmsnorm(x, w, eps, out2, rows)
    assert torch.equal(out2, out[[M - 1, 0]])


@pytest.mark.parametrize("adt,wdt,cdt", [(torch.float32,) * 3, (torch.bfloat16, torch.bfloat16, torch.float32),
                                         (torch.bfloat16, torch.bfloat16, torch.bfloat16),
                                         (torch.bfloat16, torch.float32, torch.float32)])
@pytest.mark.parametrize("M,N,K", [(1, 64, 64), (5, 100, 72), (64, 64, 16), (67, 129, 200), (130, 384, 96), (3, 1000, 320)])
def test_gemm_plain(adt, wdt, cdt, M, N, K):
    a, w = rnd(M, K, dtype=adt, seed=3), rnd(N, K, dtype=wdt, seed=4, scale=0.1)
    ref = a.float().cpu().double() @ w.float().cpu().double().T
    out = torch.full((M + 1, N), 7.0, dtype=cdt, device=DEV)  # one sentinel row behind the result
    ops().gemm_plain(a, w, out[:M])
    tol = 1e-4 if cdt == torch.float32 else 2e-2
    torch.testing.assert_close(out[:M].double().cpu(), ref, rtol=tol, atol=tol * float(ref.abs().max()))
    assert bool((out[M] == 7.0).all()), "wrote past the last row"
    if cdt == torch.float32:
        acc = rnd(M, N, seed=5)
        want = acc.cpu().double() + ref
        ops().gemm_plain(a, w, acc, accumulate=True)
        torch.testing.assert_close(acc.double().cpu(), want, rtol=1e-4, atol=1e-4 * float(want.abs().max()))


def test_gemm_plain_row_does_not_depend_on_batch():
    """A row's result is bit-identical whatever else is in the batch (32-bit path)."""
    a, w = rnd(70, 136, seed=6), rnd(90, 136, seed=7)
    full = torch.empty(70, 90, device=DEV)
    ops().gemm_plain(a, w, full)
    for r in (0, 63, 64, 69):
        one = torch.empty(1, 90, device=DEV)
        ops().gemm_plain(a[r:r + 1].contiguous(), w, one)
        assert torch.equal(one[0], full[r])


@pytest.mark.parametrize("idt", DT)
@pytest.mark.parametrize("odt", DT)
def test_swiglu(idt, odt):
    M, I, G = 5, 96, 16
    g, u = rnd(M, I, seed=8, scale=2.0).to(idt), rnd(M, I, seed=9).to(idt)
    gu = torch.stack([g.reshape(M, I // G, G), u.reshape(M, I // G, G)], 2).reshape(M, 2 * I).contiguous()
    out = torch.empty(M, I, dtype=odt, device=DEV)
    ops().swiglu(gu, out, G)
    gf, uf = g.float().cpu(), u.float().cpu()
    ref = gf / (1 + torch.exp(-gf)) * uf
    tol = 1e-6 if odt == torch.float32 else 1e-2
    torch.testing.assert_close(out.float().cpu(), ref, rtol=tol, atol=tol)


@pytest.mark.parametrize("scaling", [None, dict(rope_type="llama3", factor=32.0, low_freq_factor=1.0,
                                                high_freq_factor=4.0, original_max_position_embeddings=64)])
@pytest.mark.parametrize("D,theta", [(16, 10000.0), (48, 500000.0), (128, 500000.0)])
def test_rope_table(D, theta, scaling):
    from hipinfer_b200.parts.rotary import rope_inv_freq

    inv = rope_inv_freq(D, theta, scaling)
    ref_inv = plain.rope_inv_freq(D, theta, scaling)
    torch.testing.assert_close(inv, ref_inv, rtol=1e-6, atol=0)
    table = ops().rope_table(inv.to(DEV), 3000).cpu()
    cos, sin = plain.rope_cos_sin(list(range(3000)), ref_inv)
    torch.testing.assert_close(table[..., 0], cos, rtol=0, atol=2e-7)
    torch.testing.assert_close(table[..., 1], sin, rtol=0, atol=2e-7)


@pytest.mark.parametrize("dtype", DT)
@pytest.mark.parametrize("Hq,Hkv,D,rot", [(4, 2, 16, 16), (3, 1, 32, 32), (5, 5, 48, 24), (8, 2, 64, 64)])
def test_rope_kv_write(dtype, Hq, Hkv, D, rot):
    """Rotation against the plain formula; k, v land in the page slots named, and nowhere else."""
    from hipinfer_b200.parts.rotary import rope_inv_freq

    T, ps, n_pages = 9, 4, 7
    inv = rope_inv_freq(rot, 10000.0)
    table = ops().rope_table(inv.to(DEV), 64)
    qkv = rnd(T, (Hq + 2 * Hkv) * D, seed=10)
    pos = torch.tensor([3, 4, 5, 0, 1, 40, 41, 42, 63], dtype=torch.int32, device=DEV)
    slots = torch.tensor([12, 13, 14, 0, 1, 27, 20, 21, 5], dtype=torch.int32, device=DEV)
    q_out = torch.empty(T, Hq * D, dtype=dtype, device=DEV)
    kc = torch.full((n_pages, Hkv, ps, D), 9.0, dtype=dtype, device=DEV)
    vc = torch.full((n_pages, Hkv, ps, D), 9.0, dtype=dtype, device=DEV)
    ops().rope_kv_write(qkv, pos, slots, table, q_out, kc, vc, Hq, Hkv, D, rot, ps)
    x = qkv.cpu()
    q, k, v = x[:, :Hq * D].reshape(T, Hq, D), x[:, Hq * D:(Hq + Hkv) * D].reshape(T, Hkv, D), x[:, (Hq + Hkv) * D:].reshape(T, Hkv, D)
    cos, sin = plain.rope_cos_sin(pos.cpu().tolist(), inv)

    def rope(t):
        return torch.cat([plain.apply_rope(t[..., :rot], cos, sin), t[..., rot:]], -1)

    tol = 1e-6 if dtype == torch.float32 else 1e-2
    torch.testing.assert_close(q_out.float().cpu().reshape(T, Hq, D), rope(q), rtol=tol, atol=tol)
    kcc, vcc = kc.float().cpu(), vc.float().cpu()
    written = torch.zeros(n_pages, ps, dtype=torch.bool)
    for t in range(T):
        pg, off = int(slots[t]) // ps, int(slots[t]) % ps
        written[pg, off] = True
        torch.testing.assert_close(kcc[pg, :, off], rope(k)[t], rtol=tol, atol=tol)
        torch.testing.assert_close(vcc[pg, :, off], v[t].to(dtype).float(), rtol=0, atol=0)
    untouched = ~written[:, None, :, None].expand(n_pages, Hkv, ps, D)
    assert bool((kcc[untouched] == 9.0).all()) and bool((vcc[untouched] == 9.0).all())
    # no slot map: q only
    kc2 = kc.clone()
    ops().rope_kv_write(qkv, pos, None, table, q_out, None, None, Hq, Hkv, D, rot, ps)
    assert torch.equal(kc2, kc)


def _paged_setup(lens, Hkv, D, ps, dtype, seed, shuffle=True):
    """Random K/V per request scattered into pages in a shuffled order; returns caches, tables, per-request K, V."""
    n_pages = sum(-(-l // ps) for l in lens) + 3
    g = torch.Generator().manual_seed(seed)
    order = torch.randperm(n_pages, generator=g).tolist() if shuffle else list(range(n_pages))
    kc = torch.zeros(n_pages, Hkv, ps, D, dtype=dtype)
    vc = torch.zeros(n_pages, Hkv, ps, D, dtype=dtype)
    width = max(-(-l // ps) for l in lens)
    bt = torch.full((len(lens), width), -1, dtype=torch.int32)
    ks, vs, nxt = [], [], 0
    for r, l in enumerate(lens):
        k = torch.randn(l, Hkv, D, generator=g).to(dtype)
        v = torch.randn(l, Hkv, D, generator=g).to(dtype)
        ks.append(k.float())
        vs.append(v.float())
        for lp in range(-(-l // ps)):
            page = order[nxt]
            nxt += 1
            bt[r, lp] = page
            n = min(ps, l - lp * ps)
            kc[page, :, :n] = k[lp * ps:lp * ps + n].transpose(0, 1)
            vc[page, :, :n] = v[lp * ps:lp * ps + n].transpose(0, 1)
    return kc.to(DEV), vc.to(DEV), bt.to(DEV), ks, vs


@pytest.mark.parametrize("dtype", DT)
@pytest.mark.parametrize("Hq,Hkv,D,ps,window", [(4, 2, 16, 16, 0), (3, 1, 32, 8, 0), (10, 2, 48, 16, 0),
                                                (8, 8, 64, 16, 0), (4, 1, 128, 32, 0), (6, 2, 32, 16, 40),
                                                (4, 2, 64, 16, 300)])
def test_attention_rows(dtype, Hq, Hkv, D, ps, window):
    """Rows of several requests at once: a decode row at a long context (several key chunks),
    a portion in the middle of a sequence, a first token; a far key made to stand out."""
    lens = [700, 37, 1, 300]
    kc, vc, bt, ks, vs = _paged_setup(lens, Hkv, D, ps, dtype, 11)
    rows = [(0, 699), (1, 30), (1, 31), (1, 32), (1, 33), (1, 34), (1, 35), (1, 36), (2, 0), (3, 255), (3, 256), (3, 299)]
    T = len(rows)
    q = rnd(T, Hq * D, seed=12).to(dtype)
    # make key 3 of request 0 stand out for the first row's head 0: a far key among hundreds
    qf = q.float().cpu().reshape(T, Hq, D)
    out = torch.empty(T, Hq * D, dtype=dtype, device=DEV)
    rr = torch.tensor([r for r, _ in rows], dtype=torch.int32, device=DEV)
    pos = torch.tensor([p for _, p in rows], dtype=torch.int32, device=DEV)
    scale = 1.0 / math.sqrt(D)
    ops().attention_rows(q, kc, vc, bt, rr, pos, out, Hq, Hkv, D, ps, window, scale, max(p for _, p in rows))
    got = out.float().cpu().reshape(T, Hq, D)
    tol = 2e-5 if dtype == torch.float32 else 1e-2
    for t, (r, p) in enumerate(rows):
        ref = plain.attention_scores_softmax_values(qf[t:t + 1], ks[r][:p + 1], vs[r][:p + 1], [p], list(range(p + 1)),
                                                    window or None)
        torch.testing.assert_close(got[t:t + 1], ref, rtol=tol, atol=tol, msg=lambda m: f"row {t} {rows[t]}: {m}")


@pytest.mark.parametrize("dtype", DT)
def test_attention_rows_far_key_stands_out(dtype):
    """One early key is made to dominate the softmax of a late query: its value must come through."""
    Hq, Hkv, D, ps = 2, 1, 32, 16
    lens = [900]
    kc, vc, bt, ks, vs = _paged_setup(lens, Hkv, D, ps, dtype, 13)
    q = rnd(1, Hq * D, seed=14).to(dtype)
    qf = q.float().cpu().reshape(1, Hq, D)
    far = 5
    page, off = int(bt[0, far // ps]), far % ps
    kc[page, 0, off] = (qf[0, 0] * 4.0).to(dtype).to(DEV)  # score of this key is ~4 |q|^2/sqrt(D), far above the rest
    ks[0][far, 0] = kc[page, 0, off].float().cpu()
    out = torch.empty(1, Hq * D, dtype=dtype, device=DEV)
    ops().attention_rows(q, kc, vc, bt, torch.zeros(1, dtype=torch.int32, device=DEV),
                         torch.tensor([899], dtype=torch.int32, device=DEV), out, Hq, Hkv, D, ps, 0, 1 / math.sqrt(D), 899)
    ref = plain.attention_scores_softmax_values(qf, ks[0], vs[0], [899], list(range(900)))
    tol = 2e-5 if dtype == torch.float32 else 1e-2
    torch.testing.assert_close(out.float().cpu().reshape(1, Hq, D), ref, rtol=tol, atol=tol)
    assert float((out.float().cpu().reshape(Hq, D)[0] - vs[0][far, 0]).abs().max()) < 0.05  # head 0 ~ that key's value


def test_sample_greedy_rules():
    """Largest value, lowest index on ties, NaN above all, all -inf -> 0 (src/kernels.cuh:1883-1913)."""
    V = 5000
    l = rnd(6, V, seed=15)
    l[1, 17] = l[1, 4000] = 50.0
    l[2, 4999] = 60.0
    l[3, 123] = float("nan")
    l[3, 4500] = float("nan")
    l[4] = float("-inf")
    l[5, 0] = 70.0
    got = ops().sample(l, None, None, None).cpu().tolist()
    assert got == [plain.argmax_lowest(l[i].cpu()) for i in range(6)]
    assert got[1] == 17 and got[2] == 4999 and got[3] == 123 and got[4] == 0 and got[5] == 0


def test_sample_temperature_matches_plain_noise():
    V, R = 777, 6
    l = rnd(R, V, seed=16, scale=2.0)
    temp = torch.tensor([0.8, 0.8, 1.5, 0.0, 0.3, 0.8], dtype=torch.float32, device=DEV)
    seed = torch.tensor([4, 4, 9, 1, 2, 5], dtype=torch.int32, device=DEV)
    pos = torch.tensor([10, 11, 10, 3, 0, 10], dtype=torch.int32, device=DEV)
    got = ops().sample(l, temp, seed, pos).cpu().tolist()
    for r in range(R):
        t = float(temp[r])
        if t == 0:
            assert got[r] == plain.argmax_lowest(l[r].cpu())
            continue
        sc = plain.gumbel_scores(l[r].cpu(), t, int(seed[r]), int(pos[r]))
        assert float(sc.max() - sc[got[r]]) < 1e-4, f"row {r}: token {got[r]} is not the arg max of the noisy scores"
    # the draw depends on (seed, position) only, not on the row's place in the batch
    again = ops().sample(l[[5, 0]].contiguous(), temp[[5, 0]].contiguous(), seed[[5, 0]].contiguous(),
                         pos[[5, 0]].contiguous()).cpu().tolist()
    assert again == [got[5], got[0]]
