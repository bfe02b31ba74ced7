"""Second opinion on the paged GQA decode: flashinfer's paged-KV decode on the same page lists.

The reference runs its attention through flashinfer's ``BatchDecodeWithPagedKVCacheWrapper`` with effective
batch ``bs * H_kv``, one KV head and ``group_size`` query heads (data contract: ``indexer/context.py:117-121``,
``csrc/utils_sglang.cu:148-151`` of the reference).  The installed flashinfer is newer than the one the
reference pins, so this is a tolerance check (2e-2), not a bit-exact one.  flashinfer is the checker only: the
package never imports it.  The test skips when flashinfer cannot be imported or cannot build / load its decode
module on this machine (it compiles kernels on first use, which needs nvcc and can take minutes).
"""
import math
import os

import numpy as np
import pytest
import torch

from oracle import vortex_oracle as vo
from vortex_torch import _cabi

from _util import DevicePlan, close, to_dev

pytestmark = pytest.mark.gpu


def _flashinfer_decode(q, k, v, indptr, indices, last_len, G, D, P, scale):
    import flashinfer

    ws = torch.empty(128 * 1024 * 1024, dtype=torch.uint8, device="cuda")
    w = flashinfer.BatchDecodeWithPagedKVCacheWrapper(ws, "NHD")
    w.plan(indptr, indices, last_len, G, 1, D, P, pos_encoding_mode="NONE", q_data_type=q.dtype,
           kv_data_type=k.dtype, sm_scale=scale)
    # [rows, P, D] -> [rows, P, 1 KV head, D]
    return w.run(q, (k.unsqueeze(2), v.unsqueeze(2)))


@pytest.mark.parametrize("seq,H,G,K", [([2048, 777, 100, 16, 15, 1], 8, 2, 30), ([1024, 5000, 333], 8, 4, 64)])
def test_decode_gqa_agrees_with_flashinfer(seq, H, G, K):
    if os.environ.get("VTX_SKIP_FLASHINFER"):
        pytest.skip("disabled by VTX_SKIP_FLASHINFER")
    try:
        import flashinfer  # noqa: F401
    except Exception as e:  # pragma: no cover - depends on the machine
        pytest.skip(f"flashinfer cannot be imported: {e!r}")
    D, P, bos, eos = 128, 16, 1, 1
    prob = vo.make_paged_problem(61, seq, H, G, D, P)
    dp = DevicePlan(prob, P, H, K, bos, eos)
    d = to_dev(prob)
    scale = 1.0 / math.sqrt(D)
    sel = dp.sparse_indices.clone()
    _cabi.indexer_fused(d["q"], d["centroids"], dp.dense_indptr, dp.sparse_indptr, dp.dense_indices, sel, dp.S, K, bos,
                        eos, dp.max_pages)
    for indptr, indices in ((dp.sparse_indptr, sel), (dp.dense_indptr, dp.dense_indices)):
        ours = torch.empty_like(d["q"])
        _cabi.decode_gqa(d["q"], d["k"], d["v"], ours, indptr, indices, dp.last_page_len, dp.S, P, scale)
        try:
            theirs = _flashinfer_decode(d["q"], d["k"], d["v"], indptr[: dp.S + 1], indices, dp.last_page_len[: dp.S],
                                        G, D, P, scale)
            torch.cuda.synchronize()
        except Exception as e:  # pragma: no cover - depends on the machine
            pytest.skip(f"flashinfer's decode module is not usable here: {type(e).__name__}: {str(e)[:200]}")
        assert close(ours, theirs, 2e-2), f"max err {(ours.float() - theirs.float()).abs().max().item()}"
