import os
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (run with -m gpu on the GPU box)")


def _ensure_built():
    from gpurs_b200 import _ffi, build as builder
    import oracle

    if not _ffi.LIBRARY_PATH.exists():
        builder.build()
    if not oracle.LIBRARY_PATH.exists():
        oracle.build()


@pytest.fixture(scope="session", autouse=True)
def built_libraries():
    _ensure_built()


@pytest.fixture(scope="session")
def gpu():
    """One Gpu handle for the whole GPU session.  Fails (does not skip) when the device or the native
    library is missing: a GPU test must never pass on some other code path."""
    import gpurs_b200

    handle = gpurs_b200.Gpu(int(os.environ.get("LOCAL_RANK", "0")))
    yield handle
    status = handle.status()
    handle.close()
    assert status[0] == 0, f"a kernel reported a device-side timeout: {status}"


@pytest.fixture()
def stream(gpu):
    return gpu.stream()
