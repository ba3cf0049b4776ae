"""The tensor-core and small-batch bfloat16 kernels, each alone beside a plain float32 statement
of the same operation, at sizes other than the engine's (ragged M, N, K; both tile widths)."""
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


@pytest.mark.parametrize("tile_n", [128, 256])
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
    ob = torch.full((M + 1, N), 7.0, dtype=torch.bfloat16, device=DEV)
    fast().gemm_tc(a, w, ob[:M], fast().EPI_BF16, tile_n)
    sync_check()
    assert float((ob[:M].double() - ref).abs().max()) < 1e-2 * max(1.0, float(ref.abs().max()))
    assert bool((ob[M] == 7.0).all())


@pytest.mark.parametrize("tile_n", [128, 256])
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
