"""The operations the parts are made of, each a call into the compiled sm_100a kernels on the
current CUDA stream. Tensors are torch tensors used as typed device buffers (the reference's
binding does the same, scripts/hipinfer.py:105-190); no torch operator computes anything here.

Element types are `torch.float32` and `torch.bfloat16`. Which kernel runs is chosen from the
element types and the sizes alone (never from what else is in the batch in a way that would
change a row's arithmetic beyond rounding): the tensor-core kernels of the `fast` library for
bfloat16 operands when they take the sizes, the plain 32-bit kernels of `core` otherwise.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional

import torch

from . import library

_DT = {torch.float32: 0, torch.bfloat16: 1}
_p, _i, _l, _f = C.c_void_p, C.c_int, C.c_long, C.c_float

_SIGS = {
    "core": {
        "hb_embed": [_p, _i, _p, _p, _i, _i, _p],
        "hb_rmsnorm": [_p, _p, _i, _p, _i, _p, _i, _i, _f, _p],
        "hb_gemm_simt": [_p, _i, _l, _p, _i, _l, _p, _i, _l, _i, _i, _i, _i, _p],
        "hb_swiglu": [_p, _i, _l, _p, _i, _l, _i, _i, _i, _p],
        "hb_rope_table": [_p, _p, _i, _i, _p],
        "hb_rope_kv": [_p, _i, _l, _p, _p, _p, _p, _i, _p, _p, _i, _i, _i, _i, _i, _i, _i, _p],
        "hb_attn_rows": [_p, _i, _p, _p, _i, _p, _i, _p, _p, _p, _p, _i, _i, _i, _i, _i, _i, _f, _i, _i, _p],
        "hb_attn_merge": [_p, _p, _p, _i, _i, _i, _i, _i, _i, _i, _p, _p, _i, _p],
        "hb_sample": [_p, _l, _i, _i, _p, _p, _p, _p, _p, _p],
        "hb_convert": [_p, _i, _p, _i, _l, _p],
        "hb_feed_tokens": [_p, _p, _p, _i, _p],
    },
}
_fn_cache = {}


class KernelError(RuntimeError):
    pass


def _fn(lib_name: str, name: str):
    key = (lib_name, name)
    f = _fn_cache.get(key)
    if f is None:
        lib = library.load(lib_name)
        f = getattr(lib, name)
        f.argtypes = _SIGS[lib_name][name]
        f.restype = C.c_int
        _fn_cache[key] = f
    return f


_NO_LAUNCH = {"hb_attn_rows_workspace"}


def _call(lib_name: str, name: str, *args):
    library.launches[0] += 1
    r = _fn(lib_name, name)(*args)
    if r != 0:
        raise KernelError(library.load(lib_name).hb_last_error().decode())


def _stream() -> int:
    return library.current_stream()


def check_device_status() -> None:
    """To be called where the host has just waited for the device: raises `fast.KernelTimeout` if a kernel
    gave up on one of its bounded waits since the last call (its output is not valid), and clears the word.
    It reads one word of pinned host memory. The reference's counterpart: HI_CHECK after its calls
    (src/hip_compat.h:95-97) and the -1 of its entry points (src/api.cu:1827-1839)."""
    from . import fast

    fast.check_status()


def _dt(t: torch.Tensor) -> int:
    try:
        return _DT[t.dtype]
    except KeyError:
        raise KernelError(f"element type {t.dtype} is not supported (float32 and bfloat16 are)") from None


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _need_cuda(*ts):
    for t in ts:
        if t is not None and not t.is_cuda:
            raise KernelError("the kernels run on CUDA tensors only; there is no CPU implementation")


def _rows_contiguous(t: torch.Tensor, what: str):
    if t.dim() != 2 or t.stride(1) != 1:
        raise KernelError(f"{what}: expected a 2-D tensor with contiguous rows, got shape {tuple(t.shape)} "
                          f"strides {t.stride()}")


# ------------------------------------------------------------------------------------------
def embedding(table: torch.Tensor, tokens: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[i] = table[tokens[i]] into the float32 residual stream."""
    _need_cuda(table, tokens, out)
    T, H = out.shape
    assert out.dtype == torch.float32 and out.is_contiguous() and tokens.dtype == torch.int32
    assert table.is_contiguous() and table.shape[1] == H and tokens.numel() == T
    _call("core", "hb_embed", table.data_ptr(), _dt(table), tokens.data_ptr(), out.data_ptr(), T, H, _stream())
    return out


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor,
            rows: Optional[torch.Tensor] = None, pending: Optional["Pending"] = None) -> torch.Tensor:
    """out[i] = weight * x[rows[i] or i] / rms; x float32 [*, H], out [M, H] float32 or bfloat16.
    pending: a sum that has yet to be added into x; it is added first (in the same kernel where that applies)."""
    _need_cuda(x, weight, out, rows)
    M, H = out.shape
    if pending is not None:
        from . import fast

        if pending.out is x and pending.accumulate and fast.add_rmsnorm_slices_ok(x, pending.slices, weight, out):
            return fast.add_rmsnorm_slices(x, pending.slices, weight, eps, out, rows)
        pending.finish()
    assert x.dtype == torch.float32 and x.is_contiguous() and out.is_contiguous() and x.shape[1] == H
    assert weight.numel() == H and weight.is_contiguous()
    if rows is not None:
        assert rows.dtype == torch.int32 and rows.numel() == M
    else:
        assert x.shape[0] == M
    _call("core", "hb_rmsnorm", x.data_ptr(), weight.data_ptr(), _dt(weight), out.data_ptr(), _dt(out), _ptr(rows),
          M, H, float(eps), _stream())
    return out


def gemm_plain(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, accumulate: bool = False) -> torch.Tensor:
    """out (+)= a @ w.T with the plain 32-bit kernel: a [M, K], w [N, K], out [M, N]."""
    _need_cuda(a, w, out)
    _rows_contiguous(a, "gemm a")
    _rows_contiguous(w, "gemm w")
    _rows_contiguous(out, "gemm out")
    M, K = a.shape
    N = w.shape[0]
    assert w.shape[1] == K and out.shape == (M, N), (a.shape, w.shape, out.shape)
    _call("core", "hb_gemm_simt", a.data_ptr(), _dt(a), a.stride(0), w.data_ptr(), _dt(w), w.stride(0),
          out.data_ptr(), _dt(out), out.stride(0), M, N, K, 1 if accumulate else 0, _stream())
    return out


def swiglu(gate_up: torch.Tensor, out: torch.Tensor, group: int) -> torch.Tensor:
    """out[m, i] = silu(g) * u for a gate/up matrix [M, 2I] interleaved in groups of `group` columns."""
    _need_cuda(gate_up, out)
    _rows_contiguous(gate_up, "swiglu in")
    _rows_contiguous(out, "swiglu out")
    M, I = out.shape
    assert gate_up.shape == (M, 2 * I)
    _call("core", "hb_swiglu", gate_up.data_ptr(), _dt(gate_up), gate_up.stride(0), out.data_ptr(), _dt(out),
          out.stride(0), M, I, group, _stream())
    return out


def rope_table(inv_freq: torch.Tensor, n_pos: int) -> torch.Tensor:
    """(cos, sin) float32 [n_pos, len(inv_freq), 2] of angle = float32(p) * inv_freq[i]."""
    _need_cuda(inv_freq)
    assert inv_freq.dtype == torch.float32 and inv_freq.is_contiguous()
    half = inv_freq.numel()
    table = torch.empty(n_pos, half, 2, dtype=torch.float32, device=inv_freq.device)
    _call("core", "hb_rope_table", inv_freq.data_ptr(), table.data_ptr(), n_pos, half, _stream())
    return table


def rope_kv_write(qkv: torch.Tensor, positions: torch.Tensor, slot_map: Optional[torch.Tensor], table: torch.Tensor,
                  q_out: torch.Tensor, k_cache: Optional[torch.Tensor], v_cache: Optional[torch.Tensor], n_heads: int,
                  n_kv_heads: int, head_dim: int, rotary_dim: int, page_size: int,
                  pending: Optional["Pending"] = None) -> torch.Tensor:
    """Rotate q and k of qkv [T, (Hq + 2 Hkv) D]; q to q_out [T, Hq D]; k, v to their page slots
    (cache layout [page, Hkv, page_size, D]); slot_map None: no cache write. pending: qkv is not
    written yet, its K slices are added here (in the same kernel where that applies)."""
    _need_cuda(qkv, positions, slot_map, table, q_out, k_cache, v_cache)
    if pending is not None:
        from . import fast

        if (pending.out is qkv and not pending.accumulate and rotary_dim == head_dim and head_dim % 8 == 0
                and q_out.dtype == torch.bfloat16 and q_out.is_contiguous()
                and (slot_map is None or (k_cache.dtype == torch.bfloat16 and k_cache.is_contiguous() and v_cache.is_contiguous()))):
            return fast.rope_kv_slices(pending.slices, positions, slot_map, table, q_out, k_cache, v_cache, n_heads,
                                       n_kv_heads, head_dim, page_size)
        pending.finish()
    _rows_contiguous(qkv, "rope qkv")
    T = qkv.shape[0]
    assert qkv.shape[1] == (n_heads + 2 * n_kv_heads) * head_dim
    assert q_out.is_contiguous() and q_out.numel() == T * n_heads * head_dim
    assert table.shape[1] * 2 == rotary_dim and int(positions.numel()) == T
    if slot_map is not None:
        assert k_cache is not None and v_cache is not None and k_cache.dtype == q_out.dtype
        assert k_cache.is_contiguous() and v_cache.is_contiguous()
    _call("core", "hb_rope_kv", qkv.data_ptr(), _dt(qkv), qkv.stride(0), positions.data_ptr(), _ptr(slot_map),
          table.data_ptr(), q_out.data_ptr(), _dt(q_out), _ptr(k_cache), _ptr(v_cache), _dt(q_out), T, n_heads,
          n_kv_heads, head_dim, rotary_dim, page_size, _stream())
    return q_out


def linear_rope_kv_write(a: torch.Tensor, w: "Weight", positions: torch.Tensor, slot_map: Optional[torch.Tensor],
                         table: torch.Tensor, q_out: torch.Tensor, k_cache: Optional[torch.Tensor],
                         v_cache: Optional[torch.Tensor], n_heads: int, n_kv_heads: int, head_dim: int, rotary_dim: int,
                         page_size: int) -> bool:
    """rope_kv_write of a @ w.T in one kernel, where one takes these sizes; False: nothing was done
    (the caller projects, then rotates). The results are the same bits either way."""
    from . import fast

    if not a.is_cuda:
        return False
    return fast.linear_rope_kv(a, w, positions, slot_map, table, q_out, k_cache, v_cache, n_heads, n_kv_heads, head_dim,
                               rotary_dim, page_size)


ATTN_CHUNK = 256  # keys per split of the plain attention kernel: absolute positions, so batch-independent


def attention_rows(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, block_table: torch.Tensor,
                   row_request: torch.Tensor, positions: torch.Tensor, out: torch.Tensor, n_heads: int,
                   n_kv_heads: int, head_dim: int, page_size: int, window: int, scale: float, max_pos: int,
                   chunk: int = ATTN_CHUNK) -> torch.Tensor:
    """Causal attention of every row over its request's pages with the plain kernel.
    q, out [T, Hq D]; block_table [R, pages] int32; row_request, positions [T] int32;
    max_pos: the largest position among the rows (sizes the grid and the workspace)."""
    _need_cuda(q, k_cache, v_cache, block_table, row_request, positions, out)
    T = q.shape[0]
    assert q.is_contiguous() and out.is_contiguous() and out.dtype == q.dtype == k_cache.dtype
    assert block_table.dim() == 2 and block_table.stride(1) == 1 and block_table.dtype == torch.int32
    lib = library.load("core")
    lib.hb_attn_rows_workspace.restype = C.c_long
    lib.hb_attn_rows_workspace.argtypes = [_i, _i, _i, _i, _i]
    n_ws = lib.hb_attn_rows_workspace(T, n_heads, head_dim, int(max_pos), chunk)
    ws = torch.empty(n_ws, dtype=torch.float32, device=q.device) if n_ws else None
    _call("core", "hb_attn_rows", q.data_ptr(), _dt(q), k_cache.data_ptr(), v_cache.data_ptr(), _dt(k_cache),
          block_table.data_ptr(), block_table.stride(0), row_request.data_ptr(), positions.data_ptr(),
          out.data_ptr(), _ptr(ws), T, n_heads, n_kv_heads, head_dim, page_size, int(window), float(scale), chunk,
          int(max_pos), _stream())
    return out


def attention_workspace(T: int, n_heads: int, head_dim: int, max_pos: int, chunk: int, device):
    """The partials buffer for rows whose keys span several chunks (None when none does)."""
    lib = library.load("core")
    lib.hb_attn_rows_workspace.restype = C.c_long
    lib.hb_attn_rows_workspace.argtypes = [_i, _i, _i, _i, _i]
    n_ws = lib.hb_attn_rows_workspace(T, n_heads, head_dim, int(max_pos), chunk)
    return torch.empty(n_ws, dtype=torch.float32, device=device) if n_ws else None


def attention_merge(ws, positions, out, n_heads, head_dim, window, max_pos, chunk, row_request=None, q_len=None,
                    row_limit=0):
    """Finish rows whose keys span several chunks; rows of requests with row_limit rows or more are left alone."""
    if ws is None:
        return out
    _call("core", "hb_attn_merge", ws.data_ptr(), positions.data_ptr(), out.data_ptr(), _dt(out), out.shape[0], n_heads,
          head_dim, int(window), chunk, int(max_pos), _ptr(row_request), _ptr(q_len), int(row_limit), _stream())
    return out


def sample(logits: torch.Tensor, temperature: Optional[torch.Tensor], seed: Optional[torch.Tensor],
           position: Optional[torch.Tensor], out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """One token per row of float32 logits [R, V]: arg max (temperature 0 or None) or a
    temperature draw keyed by (seed, position) of the row."""
    _need_cuda(logits, temperature, seed, position)
    _rows_contiguous(logits, "sample logits")
    assert logits.dtype == torch.float32
    R, V = logits.shape
    if out is None:
        out = torch.empty(R, dtype=torch.int32, device=logits.device)
    if temperature is not None:
        assert temperature.dtype == torch.float32 and temperature.numel() == R
        assert seed is not None and seed.dtype in (torch.int32, torch.uint32) and seed.numel() == R
        assert position is not None and position.dtype == torch.int32 and position.numel() == R
    n = library.load("core").hb_sample_slices(V)
    ws = _sample_workspace(logits.device, R) if n > 1 else None
    _call("core", "hb_sample", logits.data_ptr(), logits.stride(0), R, V, _ptr(temperature), _ptr(seed),
          _ptr(position), out.data_ptr(), _ptr(ws), _stream())
    return out


_sample_ws = {}
_sample_ws_retired = []


def _sample_workspace(device, rows):
    """Zeroed words in which the slices of a large vocabulary meet (12 bytes a row: the kernel leaves them zero); one
    buffer per device, shared by all calls (they run one after the other on the step's stream)."""
    ws = _sample_ws.get(device)
    if ws is None or ws.numel() < 3 * rows:
        if ws is not None:
            _sample_ws_retired.append(ws)       # a captured CUDA graph may still hold the old address
        ws = _sample_ws[device] = torch.zeros(3 * max(rows, 256), dtype=torch.int32, device=device)
    return ws


def feed_tokens(tokens: torch.Tensor, src: torch.Tensor, token_map: torch.Tensor) -> torch.Tensor:
    """tokens[i] = src[token_map[i]] where token_map[i] >= 0 (all int32 on the device)."""
    _need_cuda(tokens, src, token_map)
    assert tokens.dtype == src.dtype == token_map.dtype == torch.int32 and token_map.numel() == tokens.numel()
    _call("core", "hb_feed_tokens", tokens.data_ptr(), src.data_ptr(), token_map.data_ptr(), tokens.numel(), _stream())
    return tokens


def convert(src: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    """A copy of a contiguous tensor in another element type (float32 <-> bfloat16)."""
    _need_cuda(src)
    src = src.contiguous()
    out = torch.empty(src.shape, dtype=dtype, device=src.device)
    _call("core", "hb_convert", src.data_ptr(), _dt(src), out.data_ptr(), _dt(out), src.numel(), _stream())
    return out


# ------------------------------------------------------------------------------------------
# Operations with a choice of kernel
# ------------------------------------------------------------------------------------------
class Weight:
    """A weight matrix [N, K] (K contiguous, row n produces output n, as the reference stores
    them, src/api.cu:81-83) with whatever a kernel prepared for it (tensor maps and the like)."""

    __slots__ = ("t", "prepared")

    def __init__(self, t: torch.Tensor):
        assert t.dim() == 2 and t.is_contiguous()
        self.t = t
        self.prepared = {}

    @property
    def nbytes(self) -> int:
        return self.t.numel() * self.t.element_size()

    @property
    def shape(self):
        return self.t.shape


def linear(a: torch.Tensor, w: Weight, out: torch.Tensor, accumulate: bool = False) -> torch.Tensor:
    """out (+)= a @ w.T. bfloat16 operands go to the tensor-core kernels when those take the
    sizes; everything else to the plain 32-bit kernel."""
    from . import fast

    if fast.linear(a, w, out, accumulate):
        return out
    return gemm_plain(a, w.t, out, accumulate)


def linear_swiglu(a: torch.Tensor, w_gate_up: Weight, act_out: torch.Tensor, group: int) -> torch.Tensor:
    """act_out = swiglu(a @ w_gate_up.T) for a gate/up matrix interleaved in groups of `group` rows."""
    from . import fast

    if fast.linear_swiglu(a, w_gate_up, act_out, group):
        return act_out
    gu = torch.empty(a.shape[0], w_gate_up.shape[0], dtype=torch.float32, device=a.device)
    gemm_plain(a, w_gate_up.t, gu)
    return swiglu(gu, act_out, group)


class LazyNorm:
    """The RMSNorm of residual rows that has not been computed yet: (x fp32 [T, H], weight, eps). A part that can
    fold the norm into its own first kernel (a few rows: the product's prologue) takes it as it is; any other
    calls materialize(), which runs the norm kernel. A part says that it understands one with `takes_lazy_norm`."""
    __slots__ = ("x", "weight", "eps", "dtype", "feed")

    def __init__(self, x, weight, eps, dtype, feed=None):
        self.x, self.weight, self.eps, self.dtype = x, weight, eps, dtype
        self.feed = feed       # a filled fast.NormFeed of this norm, left by the product that wrote x (or None)

    @property
    def shape(self):
        return self.x.shape

    @property
    def device(self):
        return self.x.device

    def materialize(self) -> torch.Tensor:
        out = torch.empty(self.x.shape, dtype=self.dtype, device=self.x.device)
        return rmsnorm(self.x, self.weight, self.eps, out)


def lazy_norm_applies(x: torch.Tensor, weight: torch.Tensor, dtype) -> bool:
    """Whether a consumer could fold this norm into its product: a few bf16-path rows on the device."""
    from . import fast

    return (x.is_cuda and dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and x.dtype == torch.float32
            and x.shape[0] <= fast.ROWS_MAX and not fast.PLAIN_ONLY)


def norm_linear_rope_kv_write(xn: "LazyNorm", w: "Weight", positions, slot_map, table, q_out, k_cache, v_cache, n_heads,
                              n_kv_heads, head_dim, rotary_dim, page_size) -> bool:
    """rope_kv_write of RMSNorm(x) @ w.T in one kernel for a few rows; False: nothing was done."""
    from . import fast

    if xn.feed is not None and fast.rows_scaled_qkv_rope(xn.feed, xn.x.shape[0], w.t, positions, slot_map, table, q_out, k_cache,
                                                         v_cache, n_heads, n_kv_heads, head_dim, rotary_dim, page_size):
        return True
    return fast.rows_norm_qkv_rope(xn.x, xn.weight, xn.eps, w.t, positions, slot_map, table, q_out, k_cache, v_cache, n_heads,
                                   n_kv_heads, head_dim, rotary_dim, page_size)


def norm_linear_swiglu(xn: "LazyNorm", w_gate_up: "Weight", act_out: torch.Tensor, group: int) -> bool:
    """act_out = swiglu(RMSNorm(x) @ w_gate_up.T) in one kernel for a few rows; False: nothing was done."""
    from . import fast

    if xn.feed is not None and fast.rows_scaled_swiglu(xn.feed, xn.x.shape[0], w_gate_up.t, act_out, group):
        return True
    return fast.rows_norm_swiglu(xn.x, xn.weight, xn.eps, w_gate_up.t, act_out, group)


def linear_add_rows(a: torch.Tensor, w: "Weight", out: torch.Tensor, norm_feed=None) -> bool:
    """out += a @ w.T finished in one kernel for a few rows (whole-K stripes, nothing left to add); False: nothing was done.
    norm_feed (a fast.NormFeed of the norm that reads `out` next, or None): the kernel prepares that norm on its way."""
    from . import fast

    return a.is_cuda and a.shape[0] <= fast.ROWS_MAX and fast.rows_add(a, w.t, out, norm_feed)


def make_norm_feed(weight: torch.Tensor, eps: float, rows: int):
    """A NormFeed for the norm (weight, eps) over `rows` residual rows, where the rows kernels apply; else None."""
    from . import fast

    return fast.NormFeed(weight, eps, rows) if fast.norm_feed_applies(weight, rows) else None


class Pending:
    """A product whose K slices have yet to be added: into `out` (accumulate) or as `out` itself.
    The kernel that reads the result next can add them on its way (rmsnorm and rope_kv_write take
    `pending`); anything else calls finish() first. It must be consumed before the next small
    product runs: the slices lie in scratch memory those products share."""
    __slots__ = ("slices", "out", "accumulate")

    def __init__(self, slices, out, accumulate):
        self.slices, self.out, self.accumulate = slices, out, accumulate

    def finish(self):
        from . import fast

        fast.finish_slices(self.slices, self.out, fast.EPI_ADD_F32 if self.accumulate else fast.EPI_F32)
        return self.out


def linear_deferred(a: torch.Tensor, w: Weight, out: torch.Tensor, accumulate: bool = False) -> Optional[Pending]:
    """out (+)= a @ w.T, with the last step (adding the K slices of a small product) left to the
    consumer where that applies: then a Pending comes back and `out` is not yet written. None: out is done."""
    from . import fast

    if out.dtype == torch.float32 and a.is_cuda:
        sl = fast.linear_slices(a, w)
        if sl is not None:
            return Pending(sl, out, accumulate)
    linear(a, w, out, accumulate)
    return None


def attention(q, k_cache, v_cache, batch, group: int, out, n_heads, n_kv_heads, head_dim, page_size, window, scale):
    """Attention of the step's rows over their requests' pages of cache group `group`."""
    from . import fast

    if fast.attention(q, k_cache, v_cache, batch, group, out, n_heads, n_kv_heads, head_dim, page_size, window, scale):
        return out
    return attention_rows(q, k_cache, v_cache, batch.block_tables[group], batch.row_request, batch.positions, out,
                          n_heads, n_kv_heads, head_dim, page_size, window, scale, batch.max_pos)
