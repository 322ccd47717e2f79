import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
BIN = os.path.join(ROOT, "build", "bin")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200 with `pytest -m gpu`)")


def pytest_collection_modifyitems(config, items):
    # GPU tests are skipped, not failed, when no device is visible (e.g. `pytest tests/` on a CPU box).
    try:
        import torch
        has_gpu = torch.cuda.is_available()
    except Exception:
        has_gpu = False
    if has_gpu:
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def native_build():
    """Builds the native tree once per session (no-op when it is up to date)."""
    import __graft_entry__ as entry
    entry.build()
    return BIN


def run_native(name, *args, timeout=300, env=None):
    path = os.path.join(BIN, name)
    full_env = dict(os.environ)
    if env:
        full_env.update(env)
    proc = subprocess.run([path, *args], capture_output=True, text=True, timeout=timeout, env=full_env)
    return proc
