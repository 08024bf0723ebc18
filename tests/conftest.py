import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.dirname(os.path.abspath(__file__))):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def pytest_collection_modifyitems(config, items):
    import torch
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def folders(tmp_path_factory):
    """Factory: (config name, dtype) -> model folder with random weights, made once per session."""
    from helpers import CONFIGS, write_tiny
    made = {}

    def get(name: str, dtype: str = "float32") -> str:
        key = (name, dtype)
        if key not in made:
            d = tmp_path_factory.mktemp(f"model_{name}_{dtype}")
            write_tiny(CONFIGS[name], str(d), dtype)
            made[key] = str(d)
        return made[key]
    return get
