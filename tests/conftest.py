import os
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))
os.environ.setdefault("PYTHONDONTWRITEBYTECODE", "1")

# the reference checkout, where there is one: $BSRL_REFERENCE, else a `reference` directory beside this repository
REFERENCE = Path(os.environ.get("BSRL_REFERENCE", str(ROOT.parent / "reference")))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def pytest_collection_modifyitems(config, items):
    import torch
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def golden():
    import numpy as np
    return np.load(ROOT / "tests" / "golden" / "policy_golden.npz")


@pytest.fixture(scope="session")
def native():
    """The ctypes binding; builds the library first if it is missing."""
    lib = ROOT / "beatsaberrl_b200" / "_lib" / "libbsrl.so"
    if not lib.exists():
        import shutil
        if shutil.which("nvcc") is None and not Path("/usr/local/cuda/bin/nvcc").exists():
            pytest.skip("libbsrl.so is not built and there is no nvcc to build it with")
        from beatsaberrl_b200.build import build_library
        build_library()
    from beatsaberrl_b200 import _native
    return _native


@pytest.fixture(autouse=True)
def _inference_mode_by_default():
    """The reference's callers run the rollout / evaluation forwards under torch.no_grad(); the tests do the
    same unless they ask for gradients explicitly (with torch.enable_grad())."""
    import torch
    with torch.no_grad():
        yield
