"""Weights by tensor name: what the model expects against what the folder holds.

Every part declares the tensors it needs as `ParamSpec`s (name, shape, kind). `load_weights`
compares the whole list with the file's names, shapes and element types first and raises ONE
`WeightError` that lists every missing tensor, every unexpected tensor, every wrong shape and
every wrong element type (an integer tensor under a weight's name, a float tensor where a table
of integers is expected); only then does it read. Storage policy: 16-bit floats are kept in bfloat16, integer tables become int32, and
a tensor stored in 32-bit floats stays in 32-bit.

`random_weights` / `write_random_model` are the random-weights mode: a model folder
(config.json, model.safetensors) from a configuration and a seed.

The reference's loader is positional (src/api.cu:1241-1452) and reports only a short file
(1400-1404); a missing key surfaces in its exporter as a KeyError (docs/porting-a-model.md:131).
"""
from __future__ import annotations

import hashlib
import os
from dataclasses import dataclass
from typing import Dict, Iterable, List, Optional, Sequence, Tuple

import torch

from .safetensors_io import ModelFiles, SafetensorsError, save_safetensors


@dataclass(frozen=True)
class ParamSpec:
    """One tensor a part needs. `init` tells the random-weights mode how to draw it:
    "normal" (N(0, std)), "ones" (1, plus N(0, norm_std) when asked), "zeros"."""

    name: str
    shape: Tuple[int, ...]
    init: str = "normal"
    optional: bool = False
    numbers: str = "float"       # "float": a weight (any float type in the file); "int": a table of integers


class WeightError(ValueError):
    """The folder's tensors do not fit the model. `.missing`, `.unexpected`, `.wrong_shape`, `.wrong_dtype` hold the details."""

    def __init__(self, folder, missing, unexpected, wrong_shape, other=(), wrong_dtype=()):
        self.folder, self.missing, self.unexpected = folder, list(missing), list(unexpected)
        self.wrong_shape, self.other, self.wrong_dtype = list(wrong_shape), list(other), list(wrong_dtype)
        lines = [f"{folder}: the weights do not fit the model"]
        if self.missing:
            lines.append(f"  missing ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        if self.wrong_shape:
            lines.append(f"  wrong shape ({len(self.wrong_shape)}): " + ", ".join(
                f"{n} is {list(got)}, expected {list(want)}" for n, got, want in self.wrong_shape))
        if self.wrong_dtype:
            lines.append(f"  wrong element type ({len(self.wrong_dtype)}): " + ", ".join(
                f"{n} is {got}, expected {want}" for n, got, want in self.wrong_dtype))
        for o in self.other:
            lines.append("  " + o)
        super().__init__("\n".join(lines))


def storage_dtype(dt: torch.dtype, half_as: torch.dtype = torch.bfloat16) -> torch.dtype:
    """The dtype a stored tensor is kept in. `half_as` is where IEEE half goes: bfloat16 (the
    rule), or float32 for the 32-bit engine, which would otherwise lose three bits of every weight."""
    if dt == torch.bfloat16:
        return torch.bfloat16
    if dt == torch.float16:
        return half_as
    if dt in (torch.float32, torch.float64):
        return torch.float32
    return torch.int32


_FLOATS = (torch.float16, torch.bfloat16, torch.float32, torch.float64)


def check_names(folder: str, specs: Sequence[ParamSpec], have: Dict[str, Tuple[int, ...]],
                ignore: Iterable[str] = (), dtypes: Optional[Dict[str, torch.dtype]] = None) -> None:
    """Raise the one WeightError if `have` (name -> shape) and `dtypes` (name -> element type in the file) do not fit `specs`."""
    want = {s.name: s for s in specs}
    ignore = set(ignore)
    missing = [n for n, s in want.items() if n not in have and not s.optional]
    unexpected = [n for n in have if n not in want and n not in ignore]
    wrong = [(n, have[n], s.shape) for n, s in want.items() if n in have and tuple(have[n]) != tuple(s.shape)]
    wrong_dt = []
    for n, s in want.items():
        if dtypes is None or n not in dtypes:
            continue
        is_float = dtypes[n] in _FLOATS
        if (s.numbers == "float") != is_float or dtypes[n] == torch.bool:
            wrong_dt.append((n, str(dtypes[n]).replace("torch.", ""), "a float type" if s.numbers == "float" else "an integer type"))
    if missing or unexpected or wrong or wrong_dt:
        raise WeightError(folder, sorted(missing), sorted(unexpected), sorted(wrong), wrong_dtype=sorted(wrong_dt))


def load_weights(folder: str, specs: Sequence[ParamSpec], device="cpu", ignore: Iterable[str] = (),
                 half_as: torch.dtype = torch.bfloat16) -> Dict[str, torch.Tensor]:
    """{name: tensor on `device`} for every spec, after the whole-list check."""
    try:
        files = ModelFiles(folder)
    except SafetensorsError as e:
        raise WeightError(folder, [], [], [], [str(e)]) from None
    try:
        have = {n: files.info(n)[1] for n in files.names()}
        check_names(folder, specs, have, ignore, {n: files.info(n)[0] for n in files.names()})
        out = {}
        for s in specs:
            if s.name not in have:
                continue
            t = files.get(s.name)
            out[s.name] = t.to(storage_dtype(t.dtype, half_as)).to(device)
        return out
    finally:
        files.close()


def _seed_for(seed: int, name: str) -> int:
    h = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    return int.from_bytes(h[:8], "little") & 0x7FFFFFFFFFFFFFFF


def random_weights(specs: Sequence[ParamSpec], seed: int, std: float = 0.02, norm_std: float = 0.0,
                   dtype: torch.dtype = torch.bfloat16, device="cpu") -> Dict[str, torch.Tensor]:
    """Seeded tensors for every spec: matrices N(0, std), norm weights 1 (+ N(0, norm_std)).
    Each tensor has its own stream keyed by (seed, name), so the result does not depend on
    the order of the specs. Drawn in float32 on `device`, then cast to `dtype`."""
    out = {}
    for s in specs:
        g = torch.Generator(device=device)
        g.manual_seed(_seed_for(seed, s.name))
        if s.init == "normal":
            t = torch.randn(s.shape, generator=g, dtype=torch.float32, device=device) * std
        elif s.init == "ones":
            t = torch.ones(s.shape, dtype=torch.float32, device=device)
            if norm_std:
                t = t + torch.randn(s.shape, generator=g, dtype=torch.float32, device=device) * norm_std
        elif s.init == "zeros":
            t = torch.zeros(s.shape, dtype=torch.float32, device=device)
        else:
            raise ValueError(f"ParamSpec {s.name!r}: unknown init {s.init!r}")
        out[s.name] = t.to(dtype)
    return out


def write_random_model(config, folder: str, seed: int, std: float = 0.02, norm_std: float = 0.0,
                       dtype: torch.dtype = torch.bfloat16) -> str:
    """Write config.json and model.safetensors for `config` with seeded random weights."""
    from ..config import get_architecture, save_config
    from ..parts.spec import spec_param_specs

    spec = get_architecture(config.architecture).build_spec(config)
    tensors = random_weights(spec_param_specs(spec), seed, std, norm_std, dtype)
    save_config(config, folder)
    save_safetensors(tensors, os.path.join(folder, "model.safetensors"),
                     {"format": "pt", "seed": seed, "std": std, "norm_std": norm_std})
    return folder
