import os
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
PKG = ROOT / "vortex_torch-dev_b200"
for p in (str(ROOT), str(PKG), str(ROOT / "tests")):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")
    # The host package loads the C-ABI library at import; build it when nvcc is around and it is stale.
    sys.path.insert(0, str(PKG))
    import build as vtx_build  # noqa: E402

    if vtx_build.needs_build():
        vtx_build.build()


def pytest_collection_modifyitems(config, items):
    import torch

    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def oracle():
    from oracle import vortex_oracle

    return vortex_oracle
