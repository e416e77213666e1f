"""Shared fixtures. GPU tests are marked ``gpu``; everything else runs on a CPU-only machine."""
import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import __graft_entry__ as entry  # noqa: E402

pulpnn = entry.load_package()


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")


def _has_gpu():
    try:
        import torch
        return torch.cuda.is_available()
    except Exception:
        return False


def pytest_collection_modifyitems(config, items):
    if _has_gpu():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def restatement():
    from oracle import bindings
    return bindings.Restatement()


@pytest.fixture(scope="session")
def reference32():
    from oracle import bindings
    if not bindings.have_reference(32):
        pytest.skip("compiled reference (oracle/_ref) not built on this machine")
    return bindings.CompiledReference(32)


@pytest.fixture(scope="session")
def reference64():
    from oracle import bindings
    if not bindings.have_reference(64):
        pytest.skip("compiled reference (oracle/_ref) not built on this machine")
    return bindings.CompiledReference(64)
