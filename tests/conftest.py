import os
import sys

import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
sys.path.insert(0, os.path.dirname(HERE))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def tiny_folders(tmp_path_factory):
    """Model folders of the tiny configurations, written once per session into a temporary place."""
    from tiny_configs import LONG, TINY, write_tiny_folder
    root = tmp_path_factory.mktemp("tiny-models")
    return {name: write_tiny_folder(str(root / name), name) for name in list(TINY) + list(LONG)}
