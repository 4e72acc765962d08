import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.join(ROOT, "tests")):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200)")


@pytest.fixture(scope="session")
def pkg():
    import __graft_entry__
    return __graft_entry__.load_package()


@pytest.fixture(scope="session")
def tiny_models(tmp_path_factory, pkg):
    """Tiny synthetic GGUFs in every weight scheme: {scheme: path}."""
    d = tmp_path_factory.mktemp("models")
    out = {}
    for scheme in (0, 1, 2, 3):
        out[scheme] = pkg.synth.write_gguf(str(d / f"tiny_s{scheme}.gguf"), "tiny", scheme=scheme, norm_random=True)
    return out
