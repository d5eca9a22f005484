import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")


@pytest.fixture(scope="session")
def golden_dir():
    return GOLDEN


@pytest.fixture(autouse=True)
def _switches_reread_after_test():
    """The library reads its FLAGBLAS_B200_* switches once per process.  A test that flips one (monkeypatch.setenv +
    reload_env) must not leak it: this fixture is set up before ``monkeypatch`` and so torn down after it has restored
    the environment, at which point the library is told to read the switches again."""
    yield
    mod = sys.modules.get("flagblas_b200")
    if mod is not None and hasattr(mod, "reload_env"):
        mod.reload_env()
