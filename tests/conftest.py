import os
import sys

import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
sys.path.insert(0, os.path.dirname(HERE))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


def pytest_collection_modifyitems(config, items):
    import torch
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def tiny_dirs(tmp_path_factory):
    """Model folders of the two tiny configurations, made in a temporary folder."""
    from tiny_configs import TINIES, write_tiny
    root = tmp_path_factory.mktemp("models")
    return {name: write_tiny(str(root / name), tiny) for name, tiny in TINIES.items()}
