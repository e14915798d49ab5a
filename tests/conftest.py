import os
import sys
from pathlib import Path

import pytest

REPO = Path(__file__).resolve().parents[1]
if str(REPO) not in sys.path:
    sys.path.insert(0, str(REPO))

REFERENCE = Path(os.environ.get("FXFUSION_REFERENCE") or REPO.parent / "reference")
GOLDEN = REPO / "tests" / "golden"


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


def have_reference() -> bool:
    return (REFERENCE / "py" / "fxfusion" / "passes").is_dir()


@pytest.fixture(scope="session")
def reference_py():
    if not have_reference():
        pytest.skip("reference checkout not present")
    os.environ["FXFUSION_REFERENCE_PY"] = str(REFERENCE / "py")
    from fxfusion_b200.compile_ref import _ensure_reference_importable
    _ensure_reference_importable()
    return REFERENCE / "py"


@pytest.fixture(scope="session")
def built_lib():
    """The in-tree CUDA library; built on demand where nvcc exists, never replaced by a fallback."""
    from fxfusion_b200 import _lib, build
    if not _lib.LIB_PATH.exists():
        build.build()
    return _lib.lib()


def golden_cases():
    return sorted(p.stem for p in GOLDEN.glob("*.bin"))
