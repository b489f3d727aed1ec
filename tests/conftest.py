import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
if os.path.dirname(os.path.abspath(__file__)) not in sys.path:
    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")


def pytest_collection_modifyitems(config, items):
    import torch
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def model_dirs(tmp_path_factory):
    """Model folders (config.json + model.safetensors, bfloat16) for the tiny configurations,
    written once per test session into a temporary folder."""
    from tiny_configs import TINY
    from neurogrid_b200.weights import write_random_model
    out = {}
    for name, (cfg, seed) in TINY.items():
        d = tmp_path_factory.mktemp(f"model_{name}")
        write_random_model(cfg, seed, str(d))
        out[name] = str(d)
    return out
