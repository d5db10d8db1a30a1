"""Shared pytest configuration.  `-m gpu` tests need a B200 and the built sm_100a library; everything
else runs on CPU."""
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
for p in (ROOT, ROOT / "oracle", ROOT / "tests"):
    if str(p) not in sys.path:
        sys.path.insert(0, str(p))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA GPU (B200, sm_100a)")


@pytest.fixture(scope="session")
def module():
    """The product's C-ABI shim; fails loudly when the library or the GPU is missing."""
    from triattention_b200.kernels.extension import load_extension
    return load_extension()


@pytest.fixture(scope="session")
def ref_ext():
    """The reference's own CUDA extension (oracle/_ref), or skip when it was not built."""
    import build_ref
    try:
        return build_ref.load()
    except FileNotFoundError as e:
        pytest.skip(str(e))
