import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.dirname(os.path.abspath(__file__))):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def tiny_models(tmp_path_factory):
    """Model folders of the two tiny configurations, made once per session in a temporary folder."""
    import helpers

    out = {}
    for name, (cfg, page) in helpers.TINY.items():
        d = str(tmp_path_factory.mktemp(f"tiny{name}"))
        helpers.make_model(d, cfg, seed={"A": 0, "B": 1, "C": 2}[name])
        out[name] = (d, cfg, page)
    return out
