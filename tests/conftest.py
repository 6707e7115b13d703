import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.dirname(os.path.abspath(__file__))):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (NVIDIA B200)")


def pytest_collection_modifyitems(config, items):
    import torch
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def tiny_models(tmp_path_factory):
    """Model folders of the tiny configurations with random weights, made once per run in a
    temporary folder."""
    from tiny_configs import TINY
    from zig_ai_b200.config import config_from_dict
    from zig_ai_b200.weights import write_random_model
    root = tmp_path_factory.mktemp("models")
    out = {}
    for name, (cfg_dict, seed) in TINY.items():
        d = str(root / name)
        write_random_model(config_from_dict(cfg_dict), seed, d, matrix_std="fan_in")
        out[name] = d
    return out
