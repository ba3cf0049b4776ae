"""Builds the CUDA sources under `hipinfer_b200/csrc/` for sm_100a with nvcc and loads the
shared libraries with ctypes, the way the reference binds `libhipinfer.so`
(scripts/hipinfer.py:7-8; Makefile:27-29 is its one nvcc line).

A library is compiled at its first use, and again when its sources or flags change (a stamp
file beside the .so holds their hash); what is compiled is only what was asked for. The .so
files live in `hipinfer_b200/_lib/`; when that folder cannot be written they go to a
per-user folder under the system's temporary directory. While nvcc runs, a line is printed
now and then. There is no fallback: without the library every operation raises.
"""
from __future__ import annotations

import ctypes
import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import threading
import time
from typing import Dict, List

_HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(os.path.dirname(_HERE), "csrc")

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden", "-shared", "--threads", "4"]

# library name -> sources (relative to csrc/); headers every library depends on
LIBRARIES: Dict[str, List[str]] = {
    "core": ["core.cu"],
    "fast": ["fast_entry.cu", "gemm_tc.cu", "gemm_stream.cu", "gemm_stream_consumers.cu", "gemm_rows.cu", "attention_fast.cu", "attention_prefill.cu", "attention_prefill_tc.cu", "wait_selftest.cu"],
}
HEADERS = ["common.cuh", "tc_common.cuh", "gemm_stream_static.h"]


class KernelLibraryError(RuntimeError):
    pass


_loaded: Dict[str, ctypes.CDLL] = {}
launches = [0]   # kernels launched through this package's libraries since import (a graph replay adds its own count)
_lock = threading.Lock()


def _say(msg: str) -> None:
    print(f"[hipinfer_b200] {msg}", file=sys.stderr, flush=True)


def _nvcc() -> str:
    for cand in (os.environ.get("HIPINFER_B200_NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand):
            return cand
    raise KernelLibraryError("nvcc was not found (PATH, /usr/local/cuda/bin, $HIPINFER_B200_NVCC): the CUDA "
                             "kernels cannot be compiled and there is no other implementation")


def _stamp(name: str) -> str:
    h = hashlib.sha256()
    h.update(" ".join(NVCC_FLAGS).encode())
    for rel in LIBRARIES[name] + HEADERS:
        p = os.path.join(CSRC, rel)
        if os.path.isfile(p):
            with open(p, "rb") as f:
                h.update(rel.encode() + b"\0" + f.read())
    return h.hexdigest()


def _lib_dirs() -> List[str]:
    dirs = []
    if os.environ.get("HIPINFER_B200_LIB_DIR"):
        dirs.append(os.environ["HIPINFER_B200_LIB_DIR"])
    dirs.append(os.path.join(os.path.dirname(_HERE), "_lib"))
    dirs.append(os.path.join(tempfile.gettempdir(), f"hipinfer_b200-{os.getuid()}", "_lib"))
    return dirs


def _writable_dir() -> str:
    for d in _lib_dirs():
        try:
            os.makedirs(d, exist_ok=True)
            probe = os.path.join(d, f".probe-{os.getpid()}")
            with open(probe, "w"):
                pass
            os.remove(probe)
            return d
        except OSError:
            continue
    raise KernelLibraryError(f"no writable folder for the compiled kernels among {_lib_dirs()}")


def _find_fresh(name: str, stamp: str):
    for d in _lib_dirs():
        so, st = os.path.join(d, f"libhipinfer_b200_{name}.so"), os.path.join(d, f"libhipinfer_b200_{name}.stamp")
        try:
            if os.path.isfile(so) and open(st).read().strip() == stamp:
                return so
        except OSError:
            continue
    return None


def build(name: str, verbose: bool = True) -> str:
    """Path of the up-to-date shared library `name`, compiling it if need be."""
    if name not in LIBRARIES:
        raise KernelLibraryError(f"unknown kernel library {name!r}; known: {sorted(LIBRARIES)}")
    stamp = _stamp(name)
    so = _find_fresh(name, stamp)
    if so:
        return so
    nvcc, out_dir = _nvcc(), _writable_dir()
    so = os.path.join(out_dir, f"libhipinfer_b200_{name}.so")
    tmp = os.path.join(out_dir, f".libhipinfer_b200_{name}.{os.getpid()}.so")
    srcs = [os.path.join(CSRC, s) for s in LIBRARIES[name]]
    cmd = [nvcc] + NVCC_FLAGS + ["-I", CSRC, "-o", tmp] + srcs
    if verbose:
        _say(f"compiling kernel library '{name}' for sm_100a ({len(srcs)} source file(s)) ...")
    t0 = time.time()
    env = dict(os.environ)
    env.setdefault("TMPDIR", tempfile.gettempdir())
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, env=env)
    done = threading.Event()

    def ticker():
        while not done.wait(10.0):
            if verbose:
                _say(f"  still compiling '{name}' ({time.time() - t0:.0f} s)")

    th = threading.Thread(target=ticker, daemon=True)
    th.start()
    out, _ = proc.communicate()
    done.set()
    if proc.returncode != 0:
        try:
            os.remove(tmp)
        except OSError:
            pass
        raise KernelLibraryError(f"nvcc failed for kernel library '{name}':\n{' '.join(cmd)}\n{out}")
    os.replace(tmp, so)
    with open(os.path.join(out_dir, f"libhipinfer_b200_{name}.stamp"), "w") as f:
        f.write(stamp)
    if verbose:
        _say(f"compiled '{name}' in {time.time() - t0:.0f} s -> {so}")
    return so


def load(name: str) -> ctypes.CDLL:
    """The loaded library `name` (built first if stale). Raises KernelLibraryError otherwise."""
    with _lock:
        if name in _loaded:
            return _loaded[name]
        so = build(name)
        try:
            lib = ctypes.CDLL(so)
        except OSError as e:
            raise KernelLibraryError(f"cannot load {so}: {e}") from None
        lib.hb_last_error.restype = ctypes.c_char_p
        if os.environ.get("HIPINFER_B200_PDL", "1") == "0":     # ordinary launches instead of programmatic dependent ones
            lib.hb_set_pdl(0)
        _loaded[name] = lib
        return lib


def build_all(verbose: bool = True) -> List[str]:
    return [build(n, verbose) for n in LIBRARIES]


def current_stream() -> int:
    """torch's current CUDA stream on the current device, as a raw cudaStream_t. A step launches more than a
    hundred kernels: torch.cuda.current_stream() builds a Stream object each time (several microseconds), the
    raw accessor does not."""
    import torch

    raw = getattr(torch._C, "_cuda_getCurrentRawStream", None)
    if raw is not None:
        return raw(torch._C._cuda_getDevice())
    return torch.cuda.current_stream().cuda_stream
