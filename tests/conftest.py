import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")
    config.addinivalue_line("markers", "slow: takes more than a few seconds on CPU")


def pytest_collection_modifyitems(config, items):
    import torch

    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def reference_package():
    """The reference package (``baseline/_ref``) with inert stand-ins for its uninstallable dependencies, or skip."""
    ref = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref, "deepfold3", "model")):
        pytest.skip("reference package not installed under baseline/_ref")
    from baseline.reference_arm import _stub_missing

    if ref not in sys.path:
        sys.path.insert(0, ref)
    _stub_missing()
    import deepfold3  # noqa: F401

    return ref
