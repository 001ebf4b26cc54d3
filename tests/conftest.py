import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the GPU box with -m gpu)")


@pytest.fixture(scope="session")
def built_library():
    """Builds (or reuses) libjvpfa.so; CPU tests only load it and look at its symbols."""
    from jvp_flash_attention_b200 import _lib
    if not _lib.library_path().exists():
        from jvp_flash_attention_b200 import build
        build.build()
    return _lib.lib()
