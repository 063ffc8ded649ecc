import os
import sys

import pytest

ROOT = os.path.normpath(os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))
for p in (ROOT, os.path.dirname(os.path.abspath(__file__))):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def model_dirs(tmp_path_factory):
    """Model folders of the tiny configurations, written once per session into a temp folder."""
    from harness import make_model
    from tiny_configs import TINY_A, TINY_B, TINY_C, TINY_D

    base = tmp_path_factory.mktemp("models")
    out = {}
    for name, cfg in (("A", TINY_A), ("B", TINY_B), ("C", TINY_C), ("D", TINY_D)):
        out[name] = (cfg, make_model(str(base / name), cfg, seed=11, std=0.08))
        out[name + "_small_std"] = (cfg, make_model(str(base / (name + "s")), cfg, seed=12, std=0.02))
    return out
