import os
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
PKG = ROOT / "vortex_torch-dev_b200"
for p in (str(ROOT), str(PKG), str(ROOT / "tests")):
    if p not in sys.path:
        sys.path.insert(0, p)


# VORTEX_B200_CHECKED=1 runs the suite on the checked twin of the library: every index a kernel reads and then
# uses as an address is compared with the size of the tensor it addresses, and each GPU test additionally
# asserts that no kernel reported an index out of range.  The inputs are the same valid ones: nothing here
# feeds a bad index to a GPU.
CHECKED_RUN = os.environ.get("VORTEX_B200_CHECKED", "0") not in ("", "0")


@pytest.fixture(autouse=True)
def _no_index_out_of_range(request):
    yield
    if not CHECKED_RUN or "gpu" not in request.keywords:
        return
    from vortex_torch import _cabi

    assert _cabi.CHECKED, "VORTEX_B200_CHECKED is set but the normal library is loaded"
    bits = _cabi.device_status()
    assert not bits & _cabi.STATUS_BAD_ROW, "a kernel read an index outside the tensor it addresses"


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")
    # The host package loads the C-ABI library at import; build it when nvcc is around and it is stale.
    sys.path.insert(0, str(PKG))
    import build as vtx_build  # noqa: E402

    if vtx_build.needs_build():
        vtx_build.build()
    if CHECKED_RUN and vtx_build.needs_build(checked=True):
        vtx_build.build(checked=True)


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
