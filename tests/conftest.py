import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.join(ROOT, "tests")):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def pytest_collection_modifyitems(config, items):
    try:
        import torch
        have = torch.cuda.is_available()
    except Exception:
        have = False
    if have:
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def model_dirs(tmp_path_factory):
    """Folders with random weights for the tiny configurations (made once per session, in a
    temporary place)."""
    import herbert_rs_b200 as hb
    from tiny_configs import TINY

    out = {}
    for name, cfg in TINY.items():
        d = tmp_path_factory.mktemp(f"tiny_{name}")
        hb.write_random_model(cfg, str(d), seed={"A": 11, "B": 22, "C": 33, "D": 44}.get(name, 5))
        out[name] = str(d)
    return out


def pytest_terminal_summary(terminalreporter):
    """How close the bfloat16 comparisons came to their bounds (the bound's constants rest on this)."""
    try:
        import gpu_util
    except Exception:
        return
    rec = gpu_util.RECORDS
    if not rec:
        return
    for kind in ("model", "scale"):
        r = [(e / b if b > 0 else float("inf"), w) for w, e, b, k in rec if k == kind]
        if r:
            worst = max(r)
            terminalreporter.write_line(
                f"bfloat16 comparisons ({kind}-derived bound): {len(r)}, largest error/bound {worst[0]:.3f} ({worst[1]})")
