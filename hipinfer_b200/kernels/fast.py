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
    "hb_gemm_stream": [_p, _l, _p, _l, _p, _l, _i, _i, _i, _i, _p, _l, _p, _i, _p, _p],
    "hb_gemm_stream_plan": [_i, _i, _p, _p, _p, _p],
    "hb_gemm_stream_finish": [_p, _p, _l, _i, _i, _i, _i, _p],
    "hb_add_rmsnorm_slices": [_p, _l, _p, _i, _l, _l, _p, _p, _p, _i, _i, _f, _p],
    "hb_rope_kv_slices": [_p, _i, _l, _l, _p, _p, _p, _p, _p, _p, _i, _i, _i, _i, _i, _p],
    "hb_attn_decode": [_p, _p, _p, _l, _p, _i, _p, _p, _p, _p, _p, _i, _i, _i, _i, _i, _i, _f, _i, _i, _p, _i, _p, _p, _p],
    "hb_flash_prefill": [_p, _p, _p, _p, _i, _p, _p, _p, _p, _i, _i, _i, _i, _i, _i, _i, _f, _i, _p],
    "hb_flash_prefill_supported": [_i, _i, _i],
    "hb_flash_prefill_tc": [_p, _p, _p, _l, _p, _i, _p, _p, _p, _p, _i, _i, _i, _i, _i, _i, _i, _i, _f, _i, _p, _p],
    "hb_flash_prefill_tc_supported": [_i, _i, _i, _i],
    "hb_gemm_tc_rope_kv": [_p, _l, _p, _l, _i, _i, _p, _p, _p, _p, _p, _p, _i, _i, _i, _i, _p, _p],
    "hb_attn_decode_supported": [_i, _i, _i],
    "hb_wait_selftest": [_p, _i, _p, _p],
    "hb_rows_norm_qkv_rope": [_p, _l, _p, _f, _p, _l, _i, _i, _p, _p, _p, _p, _p, _p, _i, _i, _i, _i, _p, _p],
    "hb_rows_add": [_p, _l, _p, _l, _p, _l, _i, _i, _i, _p, _p, _l, _p, _p, _p],
    "hb_rows_scaled_qkv_rope": [_p, _l, _p, _i, _f, _p, _l, _i, _i, _p, _p, _p, _p, _p, _p, _i, _i, _i, _i, _p, _p],
    "hb_rows_scaled_swiglu": [_p, _l, _p, _i, _f, _p, _l, _p, _l, _i, _i, _i, _p, _p],
    "hb_rows_norm_swiglu": [_p, _l, _p, _f, _p, _l, _p, _l, _i, _i, _i, _p, _p],
    "hb_rows_norm_supported": [_i, _i],
}
_fns = {}
_LAUNCHES = {"hb_rows_scaled_qkv_rope": 1, "hb_rows_scaled_swiglu": 1, "hb_rows_norm_qkv_rope": 1, "hb_rows_add": 1, "hb_rows_norm_swiglu": 1, "hb_gemm_tc_rope_kv": 1, "hb_gemm_stream_finish": 1, "hb_add_rmsnorm_slices": 1, "hb_rope_kv_slices": 1, "hb_gemm_tc": 1, "hb_gemm_stream": 1, "hb_attn_decode": 1, "hb_flash_prefill": 1, "hb_flash_prefill_tc": 1}
_status = None

EPI_F32, EPI_BF16, EPI_ADD_F32, EPI_SWIGLU_BF16, EPI_SLICES = 0, 1, 2, 3, 4


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
    if name in _LAUNCHES:
        library.launches[0] += _LAUNCHES[name]
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


def wait_selftest(polls: int = 4096) -> torch.Tensor:
    """Launches the one kernel whose bounded wait cannot complete (csrc/wait_selftest.cu): it gives up after
    `polls` polls, raises the status word, frees its tensor memory and returns. Returns its two result words
    (on the device): [the wait completed, the block's abort flag]. check_status() raises after it."""
    out = torch.zeros(2, dtype=torch.int32, device="cuda")
    _call("hb_wait_selftest", status_word().data_ptr(), int(polls), out.data_ptr(), _stream())
    return out


def _stream():
    return library.current_stream()


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


STREAM_MAX_ROWS = 64      # rows up to which the weight-streaming kernel is used instead of the tcgen05 kernel
_scratch = {}
_retired = []
_plans = {}


def _stream_scratch(device, ws_floats, n_counters):
    """Workspace and zeroed counters shared by all small-batch products of this device and stream
    order; they grow on demand (kernels that share them run one after the other)."""
    sc = _scratch.get(device)
    if sc is None or sc[0].numel() < ws_floats or sc[1].numel() < n_counters:
        ws = torch.empty(max(ws_floats, 16 << 20), dtype=torch.float32, device=device)
        cnt = torch.zeros(max(n_counters, 8192), dtype=torch.int32, device=device)
        if sc is not None:
            _retired.append(sc)      # a captured CUDA graph may still hold the old addresses
        sc = _scratch[device] = (ws, cnt)
    return sc


_scratch_gen = [0]       # counts the products that wrote the shared scratch: slices left there are valid until the next one


def stream_plan(N, K):
    """(kslice, ksplit, workspace floats per padded token, column blocks) of the swapped tcgen05 kernel."""
    key = ("stream", N, K)
    if key not in _plans:
        ks, sp, nb, per = C.c_int(), C.c_int(), C.c_int(), C.c_long()
        _call("hb_gemm_stream_plan", N, K, C.byref(ks), C.byref(sp), C.byref(per), C.byref(nb))
        _plans[key] = (ks.value, sp.value, per.value, nb.value)
    return _plans[key]


def gemm_stream(a, w, out, epi):
    """The swapped-operand tcgen05 weight-streaming kernel (M <= 64): see csrc/gemm_stream.cu."""
    M, K = a.shape
    N = w.shape[0]
    _, _, per_token, n_blocks = stream_plan(N, K)
    nt = 16 if M <= 16 else 32 if M <= 32 else 64
    ws, cnt = _stream_scratch(a.device, per_token * nt, n_blocks)
    _scratch_gen[0] += 1
    if stream_plan(N, K)[1] > 1 and M >= 8:
        library.launches[0] += 1     # the slices are added by a kernel of its own (counted here, launched by the call below)
    _call("hb_gemm_stream", a.data_ptr(), a.stride(0), w.data_ptr(), w.stride(0), out.data_ptr(), out.stride(0), M, N, K,
          epi, ws.data_ptr(), ws.numel(), cnt.data_ptr(), cnt.numel(), status_word().data_ptr(), _stream())
    return out


class Slices:
    """A small product a @ w.T left as the K slices it was computed in: fp32 [ksplit][rows][row_stride]
    in the scratch that all small products share, so it has to be consumed (or finished) before
    the next of them runs; `check()` raises if it was not."""
    __slots__ = ("ws", "ksplit", "slice_stride", "row_stride", "M", "N", "K", "gen")

    def check(self):
        if self.gen != _scratch_gen[0]:
            raise RuntimeError("a product left as slices was overwritten by a later product before it was consumed")


def gemm_stream_slices(a, w) -> Slices:
    """The swapped-operand kernel with the slices left for the consumer (see csrc/gemm_stream.cu, epilogue 4)."""
    M, K = a.shape
    N = w.shape[0]
    _, ksplit, per_token, n_blocks = stream_plan(N, K)
    nt = 16 if M <= 16 else 32 if M <= 32 else 64
    ws, cnt = _stream_scratch(a.device, per_token * nt, n_blocks)
    _scratch_gen[0] += 1
    _call("hb_gemm_stream", a.data_ptr(), a.stride(0), w.data_ptr(), w.stride(0), None, 0, M, N, K, EPI_SLICES,
          ws.data_ptr(), ws.numel(), cnt.data_ptr(), cnt.numel(), status_word().data_ptr(), _stream())
    sl = Slices()
    sl.ws, sl.ksplit, sl.row_stride, sl.slice_stride = ws, ksplit, n_blocks * 128, nt * n_blocks * 128
    sl.M, sl.N, sl.K, sl.gen = M, N, K, _scratch_gen[0]
    return sl


def finish_slices(sl: Slices, out, epi):
    """out per `epi` (0 to 3) from slices, as the product's own reduction would have left it."""
    sl.check()
    _call("hb_gemm_stream_finish", sl.ws.data_ptr(), out.data_ptr(), out.stride(0), sl.M, sl.N, sl.K, epi, _stream())
    return out


def add_rmsnorm_slices(x, sl: Slices, weight, eps, out, rows=None):
    """x (fp32 residual rows) += slices, out (bf16) = RMSNorm of the sum times weight: one kernel
    (csrc/gemm_stream_consumers.cu). With rows, out[i] is made from row rows[i] and x is left alone."""
    sl.check()
    M, H = out.shape
    _call("hb_add_rmsnorm_slices", x.data_ptr(), x.stride(0), sl.ws.data_ptr(), sl.ksplit, sl.slice_stride, sl.row_stride,
          weight.data_ptr(), out.data_ptr(), None if rows is None else rows.data_ptr(), M, H, float(eps), _stream())
    return out


def add_rmsnorm_slices_ok(x, sl: Slices, weight, out) -> bool:
    H = out.shape[1]
    return (x.dtype == torch.float32 and out.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and sl.N == H
            and H % 4 == 0 and H <= 8192 and x.stride(0) % 4 == 0 and out.is_contiguous() and weight.is_contiguous()
            and (x.data_ptr() | out.data_ptr() | weight.data_ptr()) % 16 == 0)


def rope_kv_slices(sl: Slices, positions, slot_map, table, q_out, k_cache, v_cache, n_heads, n_kv_heads, head_dim, page_size):
    """Rotation of q and k and the cache write on a q/k/v product left as slices (rotary over the whole head)."""
    sl.check()
    p = lambda t: None if t is None else t.data_ptr()
    _call("hb_rope_kv_slices", sl.ws.data_ptr(), sl.ksplit, sl.slice_stride, sl.row_stride, positions.data_ptr(),
          p(slot_map), table.data_ptr(), q_out.data_ptr(), p(k_cache), p(v_cache), sl.M, n_heads, n_kv_heads, head_dim,
          page_size, _stream())
    return q_out


def linear_slices(a, w):
    """a @ w.T as slices when the small-product kernel applies (a few bf16 rows), else None."""
    if a.shape[0] > STREAM_MAX_ROWS or not _tc_ok(a, w.t):
        return None
    return gemm_stream_slices(a, w.t)




def _gemm(a, w, out, epi):
    if a.shape[0] <= STREAM_MAX_ROWS:
        return gemm_stream(a, w, out, epi)
    return gemm_tc(a, w, out, epi)


def linear(a, w, out, accumulate) -> bool:
    if not _tc_ok(a, w.t):
        return False
    if out.dtype == torch.float32:
        epi = EPI_ADD_F32 if accumulate else EPI_F32
    elif out.dtype == torch.bfloat16 and not accumulate:
        epi = EPI_BF16
    else:
        return False
    _gemm(a, w.t, out, epi)
    return True




def linear_rope_kv(a, w, positions, slot_map, table, q_out, k_cache, v_cache, n_heads, n_kv_heads, head_dim, rotary_dim,
                   page_size) -> bool:
    """The q/k/v projection of more than a few rows with the rotation and the cache write in its epilogue
    (csrc/gemm_tc.cu, EPI_ROPE_KV); False where no kernel takes these sizes (heads of 64, rotated whole)."""
    if (a.shape[0] <= STREAM_MAX_ROWS or head_dim != 64 or rotary_dim != 64 or not _tc_ok(a, w.t)
            or w.shape[0] != (n_heads + 2 * n_kv_heads) * 64 or q_out.dtype != torch.bfloat16 or not q_out.is_contiguous()
            or table.dtype != torch.float32 or not table.is_contiguous()):
        return False
    if slot_map is not None and not (k_cache.dtype == torch.bfloat16 and k_cache.is_contiguous() and v_cache.is_contiguous()
                                     and v_cache.dtype == torch.bfloat16):
        return False
    p = lambda t: None if t is None else t.data_ptr()
    _call("hb_gemm_tc_rope_kv", a.data_ptr(), a.stride(0), w.t.data_ptr(), w.t.stride(0), a.shape[0], a.shape[1],
          positions.data_ptr(), p(slot_map), table.data_ptr(), q_out.data_ptr(), p(k_cache) if slot_map is not None else None,
          p(v_cache) if slot_map is not None else None, n_heads, n_kv_heads, head_dim, page_size, status_word().data_ptr(),
          _stream())
    return True


def linear_swiglu(a, w, act_out, group) -> bool:
    if group != 16 or act_out.dtype != torch.bfloat16 or not _tc_ok(a, w.t) or w.shape[0] % 32:
        return False
    _gemm(a, w.t, act_out, EPI_SWIGLU_BF16)
    return True


# ------------------------------------------------------------------------------------------
# a few token rows (csrc/gemm_rows.cu): whole-K output stripes, norm in the prologue, the layer's
# own arithmetic in the epilogue; a decoder layer of a small decode step is five kernels
# ------------------------------------------------------------------------------------------
ROWS_MAX = 8            # token rows up to which the rows kernels are used (they take up to 16; measured at the 1B shape,
                        # steps of 9 to 16 rows are 9 to 13 % faster through the split-K kernels below: two rows a warp
                        # in the norm prologue and twice the rows from L2 for every block)


ROWS_LIMIT = 16         # what the kernels themselves take (the functions below; the engine's choice is ROWS_MAX)


def _rows_w_ok(w) -> bool:
    return (not PLAIN_ONLY and w.dtype == torch.bfloat16 and w.is_contiguous() and w.shape[1] % 32 == 0
            and w.data_ptr() % 16 == 0)


def _rows_norm_ok(x, norm_w, w) -> bool:
    M, K = x.shape
    return (M <= ROWS_LIMIT and x.is_cuda and x.dtype == torch.float32 and x.stride(1) == 1 and x.stride(0) % 4 == 0
            and x.data_ptr() % 16 == 0 and norm_w.dtype == torch.bfloat16 and norm_w.is_contiguous() and norm_w.numel() == K
            and _rows_w_ok(w) and w.shape[1] == K and bool(_fn("hb_rows_norm_supported")(M, K)))


def rows_norm_qkv_rope(x, norm_w, eps, w, positions, slot_map, table, q_out, k_cache, v_cache, n_heads, n_kv_heads, head_dim,
                       rotary_dim, page_size) -> bool:
    """q, k (rotated) and v of RMSNorm(x) times the fused [q; k; v] weight for a few rows, q into q_out, k and v into their
    page slots: one kernel. False: nothing done (sizes or types it does not take)."""
    if (not _rows_norm_ok(x, norm_w, w) or head_dim % 16 or rotary_dim != head_dim
            or w.shape[0] != (n_heads + 2 * n_kv_heads) * head_dim or q_out.dtype != torch.bfloat16 or not q_out.is_contiguous()
            or table.dtype != torch.float32 or not table.is_contiguous()):
        return False
    if slot_map is not None and not (k_cache.dtype == torch.bfloat16 and v_cache.dtype == torch.bfloat16
                                     and k_cache.is_contiguous() and v_cache.is_contiguous()):
        return False
    p = lambda t: None if t is None else t.data_ptr()
    _call("hb_rows_norm_qkv_rope", x.data_ptr(), x.stride(0), norm_w.data_ptr(), float(eps), w.data_ptr(), w.stride(0),
          x.shape[0], x.shape[1], positions.data_ptr(), p(slot_map), table.data_ptr(), q_out.data_ptr(),
          p(k_cache) if slot_map is not None else None, p(v_cache) if slot_map is not None else None, n_heads, n_kv_heads,
          head_dim, page_size, status_word().data_ptr(), _stream())
    return True


class NormFeed:
    """What the product that writes the residual rows leaves for the norm that reads them next (csrc/gemm_rows.cu):
    xb [M, H] bf16 = x * norm weight (not yet divided by the row's RMS) and ssq [H / 16, 16] fp32, each 16-column
    tile's share of the rows' sums of squares. The next product takes them in place of the residual rows and applies
    1 / RMS in its epilogue: it has no norm prologue left. `filled` says whether a product has written them."""
    __slots__ = ("weight", "eps", "xb", "ssq", "filled")

    def __init__(self, weight, eps, rows):
        H = weight.numel()
        self.weight, self.eps, self.filled = weight, float(eps), False
        self.xb = torch.empty(rows, H, dtype=torch.bfloat16, device=weight.device)
        self.ssq = torch.empty(-(-H // 16), 16, dtype=torch.float32, device=weight.device)


def norm_feed_applies(weight, rows) -> bool:
    return (not PLAIN_ONLY and weight.is_cuda and weight.dtype == torch.bfloat16 and weight.is_contiguous()
            and rows <= ROWS_MAX and weight.numel() % 32 == 0)


def rows_add(act, w, out, feed: "NormFeed" = None) -> bool:
    """out (fp32) += act @ w.T for a few bf16 rows, finished in one kernel (no slices). With feed (a NormFeed for the
    norm of width N that reads `out` next) the kernel fills it as well. False: nothing done."""
    M, K = act.shape
    if (M > ROWS_LIMIT or not act.is_cuda or act.dtype != torch.bfloat16 or act.stride(1) != 1 or act.stride(0) % 8
            or act.data_ptr() % 16 or not _rows_w_ok(w) or w.shape[1] != K or out.dtype != torch.float32 or out.stride(1) != 1):
        return False
    if feed is not None and (feed.weight.numel() != w.shape[0] or feed.xb.shape[0] < M):
        feed = None
    _call("hb_rows_add", act.data_ptr(), act.stride(0), w.data_ptr(), w.stride(0), out.data_ptr(), out.stride(0), M, w.shape[0],
          K, None if feed is None else feed.weight.data_ptr(), None if feed is None else feed.xb.data_ptr(),
          0 if feed is None else feed.xb.stride(0), None if feed is None else feed.ssq.data_ptr(),
          status_word().data_ptr(), _stream())
    if feed is not None:
        feed.filled = True
    return True


def _rows_feed_ok(feed, M, w) -> bool:
    K = feed.weight.numel()
    return (feed.filled and M <= ROWS_LIMIT and _rows_w_ok(w) and w.shape[1] == K
            and bool(_fn("hb_rows_norm_supported")(M, K)))


def rows_scaled_qkv_rope(feed, M, w, positions, slot_map, table, q_out, k_cache, v_cache, n_heads, n_kv_heads, head_dim,
                         rotary_dim, page_size) -> bool:
    """rows_norm_qkv_rope from a filled NormFeed in place of the residual rows (no norm prologue). False: nothing done."""
    if (not _rows_feed_ok(feed, M, w) or head_dim % 16 or rotary_dim != head_dim
            or w.shape[0] != (n_heads + 2 * n_kv_heads) * head_dim or q_out.dtype != torch.bfloat16 or not q_out.is_contiguous()
            or table.dtype != torch.float32 or not table.is_contiguous()):
        return False
    if slot_map is not None and not (k_cache.dtype == torch.bfloat16 and v_cache.dtype == torch.bfloat16
                                     and k_cache.is_contiguous() and v_cache.is_contiguous()):
        return False
    p = lambda t: None if t is None else t.data_ptr()
    _call("hb_rows_scaled_qkv_rope", feed.xb.data_ptr(), feed.xb.stride(0), feed.ssq.data_ptr(), feed.ssq.shape[0], feed.eps,
          w.data_ptr(), w.stride(0), M, w.shape[1], positions.data_ptr(), p(slot_map), table.data_ptr(), q_out.data_ptr(),
          p(k_cache) if slot_map is not None else None, p(v_cache) if slot_map is not None else None, n_heads, n_kv_heads,
          head_dim, page_size, status_word().data_ptr(), _stream())
    return True


def rows_scaled_swiglu(feed, M, w, act_out, group) -> bool:
    """rows_norm_swiglu from a filled NormFeed in place of the residual rows. False: nothing done."""
    if (group != 16 or not _rows_feed_ok(feed, M, w) or w.shape[0] % 32 or act_out.dtype != torch.bfloat16
            or act_out.stride(1) != 1):
        return False
    _call("hb_rows_scaled_swiglu", feed.xb.data_ptr(), feed.xb.stride(0), feed.ssq.data_ptr(), feed.ssq.shape[0], feed.eps,
          w.data_ptr(), w.stride(0), act_out.data_ptr(), act_out.stride(0), M, w.shape[0], w.shape[1],
          status_word().data_ptr(), _stream())
    return True


def rows_norm_swiglu(x, norm_w, eps, w, act_out, group) -> bool:
    """act_out (bf16) = silu(gate) * up of RMSNorm(x) times a gate/up weight interleaved in groups of 16 rows. False: nothing done."""
    if (group != 16 or not _rows_norm_ok(x, norm_w, w) or w.shape[0] % 32 or act_out.dtype != torch.bfloat16
            or act_out.stride(1) != 1):
        return False
    _call("hb_rows_norm_swiglu", x.data_ptr(), x.stride(0), norm_w.data_ptr(), float(eps), w.data_ptr(), w.stride(0),
          act_out.data_ptr(), act_out.stride(0), x.shape[0], w.shape[0], x.shape[1], status_word().data_ptr(), _stream())
    return True


DECODE_CHUNK = 256      # keys per split of the decode attention kernel (absolute positions)
DECODE_CHUNK_64 = 512   # at head_dim 64 without a window: a warp walks 128 keys in two passes


def decode_chunk(head_dim: int, window: int = 0) -> int:
    """Keys per split: a constant of the layer, never of the batch (a row's split depends on its position alone).
    512 at head_dim 64 without a window (the TMA kernel walks them in two passes), else 256."""
    return DECODE_CHUNK_64 if head_dim == 64 and not window else DECODE_CHUNK


_attn_counters = {}


def _decode_counters(device, n):
    """Zeroed counters of the decode attention kernel (one per row and kv head; the kernel leaves them zero)."""
    cnt = _attn_counters.get(device)
    if cnt is None or cnt.numel() < n:
        if cnt is not None:
            _retired.append(cnt)     # a captured CUDA graph may still hold the old address
        cnt = _attn_counters[device] = torch.zeros(max(n, 16384), dtype=torch.int32, device=device)
    return cnt


def attention_decode(q, k_cache, v_cache, block_table, row_request, positions, out, n_heads, n_kv_heads, head_dim,
                     page_size, window, scale, max_pos, chunk=None, q_len=None, row_limit=0, ctx_len=None):
    """The bf16 row-attention kernel itself (see csrc/attention_fast.cu); rows whose keys span several
    chunks are finished inside it. With q_len (int32 per request) rows of requests with row_limit
    rows or more are skipped. row_request None: row t is the only row of request t (a decode-only
    step). ctx_len (int32 per request): the tokens in the cache before this
    step; with it the kernel asks for their keys before the kernel ahead of it has ended, so
    positions, tables and ctx_len must then be in place before that kernel starts."""
    from . import ops

    T = q.shape[0]
    chunk = chunk or decode_chunk(head_dim, int(window))
    ws = ops.attention_workspace(T, n_heads, head_dim, max_pos, chunk, q.device)
    cnt = None if ws is None else _decode_counters(q.device, T * n_kv_heads)
    _call("hb_attn_decode", q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), k_cache.shape[0], block_table.data_ptr(),
          block_table.stride(0), None if row_request is None else row_request.data_ptr(), positions.data_ptr(), out.data_ptr(),
          None if ws is None else ws.data_ptr(), None if cnt is None else cnt.data_ptr(), T, n_heads, n_kv_heads,
          head_dim, page_size, int(window), float(scale), chunk, int(max_pos),
          None if q_len is None else q_len.data_ptr(), int(row_limit), None if ctx_len is None else ctx_len.data_ptr(),
          status_word().data_ptr(), _stream())
    return out


def attention_decode_supported(n_heads, n_kv_heads, head_dim) -> bool:
    return bool(_fn("hb_attn_decode_supported")(n_heads, n_kv_heads, head_dim))


def flash_prefill_supported(n_heads, n_kv_heads, head_dim) -> bool:
    return bool(_fn("hb_flash_prefill_supported")(n_heads, n_kv_heads, head_dim))


def flash_prefill(q, k_cache, v_cache, block_table, q_start, q_len, ctx_len, out, max_q_len, n_heads, n_kv_heads,
                  head_dim, page_size, window, scale, min_rows=1):
    """The flash kernel for prompt portions itself (see csrc/attention_prefill.cu): per request
    q_start, q_len, ctx_len (int32 on the device); requests with fewer than min_rows rows are skipped."""
    _call("hb_flash_prefill", q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), block_table.data_ptr(),
          block_table.stride(0), q_start.data_ptr(), q_len.data_ptr(), ctx_len.data_ptr(), out.data_ptr(),
          q_len.numel(), int(max_q_len), n_heads, n_kv_heads, head_dim, page_size, int(window), float(scale),
          int(min_rows), _stream())
    return out




def flash_prefill_tc_supported(n_heads, n_kv_heads, head_dim, page_size) -> bool:
    return bool(_fn("hb_flash_prefill_tc_supported")(n_heads, n_kv_heads, head_dim, page_size))


def flash_prefill_tc(q, k_cache, v_cache, block_table, q_start, q_len, ctx_len, out, max_q_len, n_heads, n_kv_heads,
                     head_dim, page_size, window, scale, min_rows=1):
    """The tcgen05 flash kernel for prompt portions (see csrc/attention_prefill_tc.cu); arguments as flash_prefill."""
    _call("hb_flash_prefill_tc", q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), k_cache.shape[0],
          block_table.data_ptr(), block_table.stride(0), q_start.data_ptr(), q_len.data_ptr(), ctx_len.data_ptr(),
          out.data_ptr(), q.shape[0], q_len.numel(), int(max_q_len), n_heads, n_kv_heads, head_dim, page_size, int(window),
          float(scale), int(min_rows), status_word().data_ptr(), _stream())
    return out


FLASH_MIN_ROWS = 16     # portions of at least this many rows go to the flash kernel, shorter ones to the row kernel


def attention(q, k_cache, v_cache, batch, group, out, n_heads, n_kv_heads, head_dim, page_size, window, scale) -> bool:
    if PLAIN_ONLY or q.dtype != torch.bfloat16 or not attention_decode_supported(n_heads, n_kv_heads, head_dim):
        return False
    use_flash = flash_prefill_supported(n_heads, n_kv_heads, head_dim) and batch.max_q_len >= FLASH_MIN_ROWS
    need_rows = not use_flash or min(batch.h_q_len) < FLASH_MIN_ROWS
    bt = batch.block_tables[group]
    if use_flash:
        tc = flash_prefill_tc_supported(n_heads, n_kv_heads, head_dim, page_size)    # else: warp MMAs (other page sizes)
        (flash_prefill_tc if tc else flash_prefill)(q, k_cache, v_cache, bt, batch.req_q_start, batch.req_q_len,
                                                    batch.req_ctx_len, out, batch.max_q_len, n_heads, n_kv_heads,
                                                    head_dim, page_size, window, scale, FLASH_MIN_ROWS)
    if need_rows:
        # a step of single decode rows: row t is request t, which the kernel need not look up
        rows_are_requests = batch.max_q_len == 1 and batch.n_rows == batch.n_requests
        attention_decode(q, k_cache, v_cache, bt, None if rows_are_requests else batch.row_request, batch.positions, out, n_heads, n_kv_heads,
                         head_dim, page_size, window, scale, batch.max_pos,
                         q_len=batch.req_q_len if use_flash else None, row_limit=FLASH_MIN_ROWS,
                         ctx_len=batch.req_ctx_len)
    return True
