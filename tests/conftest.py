import os
import sys

import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
for p in (ROOT, HERE):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200 with -m gpu)")


def pytest_collection_modifyitems(config, items):
    import torch

    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


def pytest_terminal_summary(terminalreporter):
    """The measured error of the logits comparisons: per configuration and precision, the largest
    |difference| over the largest |logit| of a request under each plan (worst request)."""
    try:
        import tiny
    except Exception:
        return
    worst = {}
    for (config, plan), dtype, rel in tiny.MEASURED:
        plans = worst.setdefault((config, dtype), {})
        plans[plan] = max(plans.get(plan, 0.0), rel)
    if worst:
        terminalreporter.write_line("logits against the plain implementation, largest |diff| / largest |logit| (bound: "
                                    + ", ".join(f"{k} {v:.1e}" for k, v in tiny.TOL.items()) + "):")
        for (config, dtype), plans in sorted(worst.items()):
            terminalreporter.write_line(f"  {config:22s} {dtype:9s} " + "  ".join(f"{p or 'all'} {r:.1e}" for p, r in sorted(plans.items())))
