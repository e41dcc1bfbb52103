"""pytest configuration: the `gpu` marker and the build of the CPU checker library."""
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests"))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (run with -m gpu on the GPU box)")


@pytest.fixture(scope="session")
def oracle_lib():
    """oracle/libsofie_oracle.so, built on first use (plain gcc, a second or two)."""
    so = ROOT / "oracle" / "libsofie_oracle.so"
    src = ROOT / "oracle" / "sofie_oracle.c"
    if not so.exists() or so.stat().st_mtime < src.stat().st_mtime:
        subprocess.run(["make", "-C", str(ROOT / "oracle"), "oracle"], check=True, capture_output=True)
    return so


@pytest.fixture(scope="session")
def b200_lib():
    """libsofie_b200.so must already be built (python -m sofie_b200.build); no fallback."""
    from sofie_b200 import lib
    return lib.load()
