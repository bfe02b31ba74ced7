"""The checked twin of the library (``VORTEX_B200_CHECKED=1``): that its index checks are armed.

Run the whole GPU suite with that variable set to compare every row id, ``loc`` entry and request slot of every
parity case with the size of the tensor it addresses (``conftest.py`` asserts after each test that nothing was
reported).  The tests here only show that the limits reach the device with the values the wrappers derive from
the tensors; all inputs are valid ones, and the status word must stay clear.
"""
import math

import pytest
import torch

from oracle import vortex_oracle as vo
from vortex_torch import _cabi

from _util import DevicePlan, close, to_dev

pytestmark = [pytest.mark.gpu, pytest.mark.skipif(not _cabi.CHECKED, reason="the normal library is loaded")]


def test_limits_follow_the_tensors_of_each_call():
    seq, H, G, D, P, K = [700, 33, 2048], 4, 2, 128, 16, 8
    prob = vo.make_paged_problem(71, seq, H, G, D, P)
    dp = DevicePlan(prob, P, H, K, 1, 1)
    d = to_dev(prob)
    rows = d["k"].shape[0]
    out = torch.empty_like(d["q"])
    _cabi.decode_gqa(d["q"], d["k"], d["v"], out, dp.dense_indptr, dp.dense_indices, dp.last_page_len, dp.S, P,
                     1.0 / math.sqrt(D))
    assert _cabi.checked_limits() == (rows, -1, -1, -1)
    sel = dp.sparse_indices.clone()
    _cabi.indexer_fused(d["q"], d["centroids"], dp.dense_indptr, dp.sparse_indptr, dp.dense_indices, sel, dp.S, K, 1, 1,
                        dp.max_pages)
    assert _cabi.checked_limits() == (-1, d["centroids"].shape[0], -1, -1)
    loc = torch.as_tensor([int(prob["req_to_token"][r, seq[r] - 1]) for r in range(len(seq))], dtype=torch.int64).cuda()
    nk = torch.zeros(len(seq), H, D, dtype=torch.bfloat16, device="cuda")
    _cabi.sparse_layer_fused(d["q"], d["centroids"], d["k"], d["v"], out, dp.dense_indptr, dp.sparse_indptr,
                             dp.dense_indices, sel, dp.last_page_len, dp.S, P, K, 1, 1, dp.max_pages,
                             1.0 / math.sqrt(D), nk, nk.clone(), loc)
    assert _cabi.checked_limits() == (rows, d["centroids"].shape[0], rows // H * P, -1)
    want = vo.decode_gqa(prob["q"], prob["k"], prob["v"], dp.oracle(prob)["dense_kv_indptr"],
                         dp.oracle(prob)["dense_kv_indices"], dp.oracle(prob)["kv_last_page_len"])
    _cabi.decode_gqa(d["q"], to_dev(prob)["k"], to_dev(prob)["v"], out, dp.dense_indptr, dp.dense_indices,
                     dp.last_page_len, dp.S, P, 1.0 / math.sqrt(D))
    assert close(out, want, 2e-2)
    assert _cabi.device_status() == 0
