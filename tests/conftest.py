"""Test configuration: import paths for the package and the oracle, the `gpu` marker, and an in-tree build of the
C-ABI library when it is missing."""
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
PACKAGE_ROOT = ROOT / "zig-flash-attn_b200"
for path in (PACKAGE_ROOT, ROOT / "oracle", ROOT / "tests", ROOT):
    if str(path) not in sys.path:
        sys.path.insert(0, str(path))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")
    library = PACKAGE_ROOT / "zigfa" / "libb200fa.so"
    if not library.exists():
        import importlib.util

        spec = importlib.util.spec_from_file_location("b200fa_build", PACKAGE_ROOT / "build.py")
        module = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(module)
        module.build()


@pytest.fixture(autouse=True)
def _device_status_is_clean(request):
    """After every GPU test: no kernel wait may have run out of time."""
    yield
    if "gpu" in request.keywords:
        from zigfa._impl import lib

        assert lib.library().b200fa_device_status() == 0, "a kernel wait timed out (device status word set)"
