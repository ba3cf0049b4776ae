"""hb_gemm_stream_static, the decode-step matrix product for callers that cannot allocate
device memory (a plug-in inside an application that owns the GPU's memory, a real-time path
where cudaMalloc is forbidden, a process whose memory budget is spent): its split-K scratch
lives in arrays inside the library instead of a workspace from the caller.

The test calls it through its exported C symbol, twice in a row, and compares with the
ordinary entry point (hb_gemm_stream with a caller-allocated workspace) on the same inputs.
Everything the call touches is allocated before it; the call itself must not allocate: the
driver's count of free device memory (cudaMemGetInfo, which sees every allocation on the GPU,
the library's own included) is the same after the calls as before them. It also checks that a
product beyond the arrays' size, a bad epilogue code and a missing status word are refused with
a message before anything is queued. This file is collected
last so that a run that stops at the first failure has already run every other test.
"""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _lib():
    from hipinfer_b200.kernels import fast, library

    lib = library.load("fast")
    fn = lib.hb_gemm_stream_static
    fn.restype = C.c_int
    fn.argtypes = [C.c_void_p, C.c_long, C.c_void_p, C.c_long, C.c_void_p, C.c_long, C.c_int, C.c_int, C.c_int, C.c_int,
                   C.c_void_p, C.c_void_p]
    return lib, fn, fast


@pytest.mark.parametrize("M,N,K,epi", [(8, 3072, 2048, 0), (1, 2048, 8192, 2), (16, 1024, 2048, 3), (33, 384, 520, 1)])
def test_static_scratch_matches_the_ordinary_entry_point(M, N, K, epi):
    lib, fn, fast = _lib()
    g = torch.Generator().manual_seed(M + N)
    a = torch.randn(M, K, generator=g).to(torch.bfloat16).to(DEV)
    w = (torch.randn(N, K, generator=g) * 0.05).to(torch.bfloat16).to(DEV)
    out_dtype = torch.bfloat16 if epi in (1, 3) else torch.float32
    out_cols = N // 2 if epi == 3 else N
    base = torch.randn(M, out_cols, generator=g).to(out_dtype).to(DEV)
    want = base.clone()
    fast.gemm_stream(a, w, want, epi)                       # the existing entry point, workspace from the caller
    ref = a.float() @ w.float().T
    status = fast.status_word()
    stream = torch.cuda.current_stream().cuda_stream
    outs = [base.clone(), base.clone()]                     # allocated before the calls
    warm = base.clone()                                     # a first call has looked up the arrays' addresses and loaded the kernel
    assert fn(a.data_ptr(), a.stride(0), w.data_ptr(), w.stride(0), warm.data_ptr(), warm.stride(0), M, N, K, epi,
              status.data_ptr(), stream) == 0, lib.hb_last_error().decode()
    torch.cuda.synchronize()
    before, before_torch = torch.cuda.mem_get_info()[0], torch.cuda.memory_allocated()
    for out in outs:                                        # two calls in a row share the arrays
        rc = fn(a.data_ptr(), a.stride(0), w.data_ptr(), w.stride(0), out.data_ptr(), out.stride(0), M, N, K, epi,
                status.data_ptr(), stream)
        assert rc == 0, lib.hb_last_error().decode()
    torch.cuda.synchronize()
    fast.check_status()
    assert torch.cuda.mem_get_info()[0] == before, "free device memory changed: something allocated"
    assert torch.cuda.memory_allocated() == before_torch
    for out in outs + [warm]:
        assert torch.equal(out, want)
    if epi == 0:                                            # and the ordinary entry point itself is right
        assert float((want - ref).abs().max()) < 2e-5 * float(ref.abs().max()) * K ** 0.5


def test_sizes_beyond_the_static_arrays_are_refused():
    lib, fn, fast = _lib()
    M, N, K = 64, 16384, 2048                               # 3 slices x 128 blocks x 128 x 64 floats > 4 MiB
    a = torch.zeros(M, K, dtype=torch.bfloat16, device=DEV)
    w = torch.zeros(N, K, dtype=torch.bfloat16, device=DEV)
    out = torch.full((M, N), 7.0, dtype=torch.float32, device=DEV)
    rc = fn(a.data_ptr(), K, w.data_ptr(), K, out.data_ptr(), N, M, N, K, 0, fast.status_word().data_ptr(),
            torch.cuda.current_stream().cuda_stream)
    assert rc != 0
    msg = lib.hb_last_error().decode()
    assert "static array holds" in msg and "need" in msg
    small_a, small_w = a[:8], w[:256]
    for epi, status_ptr, frag in ((4, fast.status_word().data_ptr(), "epilogue"), (7, fast.status_word().data_ptr(), "epilogue"),
                                  (0, None, "status")):
        rc = fn(small_a.data_ptr(), K, small_w.data_ptr(), K, out.data_ptr(), N, 8, 256, K, epi, status_ptr,
                torch.cuda.current_stream().cuda_stream)
        assert rc != 0 and frag in lib.hb_last_error().decode()
    torch.cuda.synchronize()
    assert bool((out == 7.0).all()), "a refused call must not launch anything"
