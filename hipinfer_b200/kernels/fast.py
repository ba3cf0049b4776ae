"""Dispatch to the tensor-core kernels of the `fast` library (bfloat16 operands). Each function
returns False when its kernel does not take the element types or sizes; the caller then uses
the plain kernel. Set HIPINFER_B200_PLAIN=1 to force the plain kernels everywhere.

The kernels' waits are bounded; one that runs out sets a status word in pinned host memory
that `check_status()` reads after a synchronisation.
"""
from __future__ import annotations

import ctypes as C
import os

import torch

from . import library

PLAIN_ONLY = os.environ.get("HIPINFER_B200_PLAIN", "0") == "1"

_p, _i, _l, _f = C.c_void_p, C.c_int, C.c_long, C.c_float
_SIGS = {
    "hb_gemm_tc": [_p, _l, _p, _l, _p, _l, _i, _i, _i, _i, _i, _p, _p],
}
_fns = {}
_status = None

EPI_F32, EPI_BF16, EPI_ADD_F32, EPI_SWIGLU_BF16 = 0, 1, 2, 3


class KernelTimeout(RuntimeError):
    """A bounded wait inside a kernel ran out: the kernel returned early and its output is not valid."""


def _fn(name):
    f = _fns.get(name)
    if f is None:
        lib = library.load("fast")
        f = getattr(lib, name)
        f.argtypes = _SIGS[name]
        f.restype = C.c_int
        _fns[name] = f
    return f


def _call(name, *args):
    if _fn(name)(*args) != 0:
        from .ops import KernelError

        raise KernelError(library.load("fast").hb_last_error().decode())


def status_word() -> torch.Tensor:
    """One int32 in pinned host memory that the device can write (the same address under unified addressing)."""
    global _status
    if _status is None:
        _status = torch.zeros(4, dtype=torch.int32, pin_memory=True)
    return _status


def check_status() -> None:
    """Call after a synchronisation: raises if a kernel gave up on a wait since the last check."""
    if _status is not None and int(_status[0]) != 0:
        _status[0] = 0
        raise KernelTimeout("a tensor-core kernel gave up on a bounded wait (TMA or MMA pipeline); its output is invalid")


def _stream():
    return torch.cuda.current_stream().cuda_stream


def _tc_ok(a, w) -> bool:
    return (not PLAIN_ONLY and a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and a.shape[1] % 8 == 0
            and a.stride(0) % 8 == 0 and w.stride(0) % 8 == 0 and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def gemm_tc(a, w, out, epi, tile_n=0):
    """The tcgen05 kernel itself: out per `epi` (see csrc/gemm_tc.cu)."""
    M, K = a.shape
    N = w.shape[0]
    _call("hb_gemm_tc", a.data_ptr(), a.stride(0), w.data_ptr(), w.stride(0), out.data_ptr(), out.stride(0), M, N, K,
          epi, tile_n, status_word().data_ptr(), _stream())
    return out


def linear(a, w, out, accumulate) -> bool:
    if not _tc_ok(a, w.t):
        return False
    if out.dtype == torch.float32:
        epi = EPI_ADD_F32 if accumulate else EPI_F32
    elif out.dtype == torch.bfloat16 and not accumulate:
        epi = EPI_BF16
    else:
        return False
    gemm_tc(a, w.t, out, epi)
    return True


def linear_swiglu(a, w, act_out, group) -> bool:
    if group != 16 or act_out.dtype != torch.bfloat16 or not _tc_ok(a, w.t) or w.shape[0] % 32:
        return False
    gemm_tc(a, w.t, act_out, EPI_SWIGLU_BF16)
    return True


def attention(q, k_cache, v_cache, batch, group, out, n_heads, n_kv_heads, head_dim, page_size, window, scale) -> bool:
    return False
