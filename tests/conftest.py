import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.join(ROOT, "tests")):
    if p not in sys.path:
        sys.path.insert(0, p)


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
    """Model folders (config.json + model.safetensors) of the tiny configurations, made once per run."""
    import helpers
    root = tmp_path_factory.mktemp("models")
    return {name: helpers.make_model_dir(str(root / name), name) for name in helpers.TINY}


@pytest.fixture()
def cpu_ops_installed(monkeypatch):
    import cpu_ops
    cpu_ops.install(monkeypatch)
    return cpu_ops
