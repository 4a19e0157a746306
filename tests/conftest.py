import os
import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))
GOLDEN = Path(__file__).resolve().parent / "golden"


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (sm_100a) GPU; run with -m gpu")


def pytest_collection_modifyitems(config, items):
    # the shared library is built once for the whole session (cross-compiles without a GPU)
    from x17ai_b200 import build
    build.build()
    build.build_kernel_objects()


@pytest.fixture(scope="session")
def lib():
    from x17ai_b200 import _lib
    return _lib.load()


@pytest.fixture()
def stream():
    """A stream opened through the C ABI; after the test, no kernel may have given up a wait."""
    from x17ai_b200 import device
    s = device.CudaStream(0)
    yield s
    status = s.read_status()
    s.close()
    assert status == [0, 0, 0, 0], f"device status words after the test: {status}"


def load_golden(name):
    g = np.load(GOLDEN / f"{name}.npz")
    seq, dm, hd, nh, fw, win = [int(v) for v in g["config"]]
    return g, dict(S=seq, Dm=dm, D=hd, H=nh, F=fw, W=win)


def code_hist(a, b):
    d = np.abs(a.astype(np.int32) - b.astype(np.int32))
    return np.bincount(d.ravel(), minlength=8)


def reference_build_missing(what: str):
    """oracle/_ref (the reference's own kernels compiled for sm_100a by oracle/build_ref.py) is git-ignored: a
    fresh clone has none until the recipe has run. Where a checkout of the reference is declared
    (X17AI_REFERENCE) its absence is a failure, elsewhere a skip."""
    import os
    import pytest
    msg = f"oracle/_ref has no {what} (python oracle/build_ref.py <reference checkout>)"
    if os.environ.get("X17AI_REFERENCE"):
        pytest.fail(msg + ": X17AI_REFERENCE is set, so __graft_entry__.build() should have made it")
    pytest.skip(msg)
