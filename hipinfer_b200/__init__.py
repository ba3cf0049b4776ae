"""hipinfer_b200: a small, whole, single-GPU inference engine for NVIDIA B200 (sm_100a).

    from hipinfer_b200 import Engine
    tokens = Engine("model_dir").generate([1, 2, 3], 16)
"""
from . import config, weights, cache, parts, models  # noqa: F401  (models registers the architectures)

__version__ = "0.1.0"


def __getattr__(name):
    if name in ("Engine", "SamplingParams"):
        from .engine import api

        return getattr(api, name)
    raise AttributeError(name)
