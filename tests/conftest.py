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
