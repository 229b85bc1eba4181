import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.dirname(os.path.abspath(__file__))):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


def pytest_collection_modifyitems(config, items):
    # a test marked gpu is skipped where there is no device, so a plain `pytest tests` passes anywhere
    import torch
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture
def fake_backend():
    """The torch stand-in for the CUDA extension, for tests of the host-side logic."""
    import fake_ops
    from vt_transformer_b200 import ops
    ops.use_backend(fake_ops)
    yield fake_ops
    ops.use_backend(None)


@pytest.fixture(scope="session")
def folders(tmp_path_factory):
    """Model folders of the tiny configurations with random weights, made once a session in a
    temporary place."""
    import helpers
    made = {}

    def get(name):
        if name not in made:
            made[name] = helpers.make_folder(name, str(tmp_path_factory.mktemp(f"model_{name}")))
        return made[name]

    return get
