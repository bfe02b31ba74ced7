"""Long segments: the scan of one (request, head) segment split over several CTAs, segments with more
candidates than the register sort holds, and the status word raised by an understated page bound.

Selections must be the oracle's bit for bit in every form; attention outputs within 2e-2.
"""
import math

import numpy as np
import pytest
import torch

from oracle import vortex_oracle as vo
from vortex_torch import _cabi

from _util import DevicePlan, close, to_dev

pytestmark = pytest.mark.gpu
BF16_TOL = 2e-2


def _problem(seed, seq, H, G, D, P, K, bos, eos):
    prob = vo.make_paged_problem(seed, seq, H, G, D, P)
    dp = DevicePlan(prob, P, H, K, bos, eos)
    ref = dp.oracle(prob)
    vo.forward_indexer(prob["q"], prob["centroids"], ref, K, bos, eos)
    return prob, dp, ref


def _workspace(dp, K, bos, eos, poison=True):
    n = _cabi.sparse_layer_workspace_bytes(dp.S, dp.max_pages, K, bos, eos)
    assert n > 0, "the case is meant to need a split"
    ws = torch.zeros(n // 4, dtype=torch.int32, device="cuda")
    if poison:  # only the arrival counters (the first eff_bs words, padded to 256 bytes) have to start at zero
        ws[(dp.S * 4 + 255) // 256 * 64:] = 0x7F7F7F7F
    return ws


@pytest.mark.parametrize("seq,H,G,K", [
    ([32768, 9000, 8208, 1024, 600, 17], 8, 4, 64),   # ragged batch incl. the longest request of config 3
    ([16 * 771, 16 * 770], 8, 2, 30),                 # just above / at one chunk of 768 candidates (small batches)
    ([8192 + 16 * 3, 8192] + [40] * 58, 8, 2, 30),    # 480 segments: chunks of 512; just above / at one chunk
    ([20000, 16400], 2, 8, 30),
])
def test_sparse_layer_split_segments_match_oracle_and_unsplit(seq, H, G, K):
    D, P, bos, eos = 128, 16, 1, 1
    prob, dp, ref = _problem(41, seq, H, G, D, P, K, bos, eos)
    d = to_dev(prob)
    ns = int(ref["sparse_kv_indptr"][-1])
    want = vo.decode_gqa(prob["q"], prob["k"], prob["v"], ref["sparse_kv_indptr"], ref["sparse_kv_indices"],
                         ref["kv_last_page_len"])
    scale = 1.0 / math.sqrt(D)
    sel0 = dp.sparse_indices.clone()
    out0 = torch.full_like(d["q"], float("nan"))
    _cabi.sparse_layer_fused(d["q"], d["centroids"], d["k"], d["v"], out0, dp.dense_indptr, dp.sparse_indptr,
                             dp.dense_indices, sel0, dp.last_page_len, dp.S, P, K, bos, eos, dp.max_pages, scale)
    np.testing.assert_array_equal(sel0.cpu().numpy()[:ns], ref["sparse_kv_indices"])
    assert close(out0, want, BF16_TOL)
    ws = _workspace(dp, K, bos, eos)
    for _ in range(3):  # the arrival counters must come back to zero after every launch
        sel1 = dp.sparse_indices.clone()
        out1 = torch.full_like(d["q"], float("nan"))
        _cabi.sparse_layer_fused(d["q"], d["centroids"], d["k"], d["v"], out1, dp.dense_indptr, dp.sparse_indptr,
                                 dp.dense_indices, sel1, dp.last_page_len, dp.S, P, K, bos, eos, dp.max_pages, scale,
                                 workspace=ws)
        np.testing.assert_array_equal(sel1.cpu().numpy()[:ns], ref["sparse_kv_indices"])
        assert torch.equal(out1.view(torch.int16), out0.view(torch.int16))
        assert int(ws[:dp.S].abs().sum().item()) == 0
    assert _cabi.device_status() == 0


def test_sparse_layer_split_with_token_append():
    """Split segments with the new-token write: the CTA that merges sees the token another CTA wrote."""
    seq, H, G, D, P, K, bos, eos = [16384, 32768, 2048, 9008], 8, 2, 128, 16, 30, 1, 1
    prob, dp, ref = _problem(43, seq, H, G, D, P, K, bos, eos)
    bs = len(seq)
    loc = torch.as_tensor([int(prob["req_to_token"][r, seq[r] - 1]) for r in range(bs)], dtype=torch.int64).cuda()
    g = torch.Generator().manual_seed(5)
    nk = torch.randn(bs, H, D, generator=g).bfloat16().cuda()
    nv = torch.randn(bs, H, D, generator=g).bfloat16().cuda()
    scale = 1.0 / math.sqrt(D)
    res = []
    for split in (False, True):
        d = to_dev(prob)
        k, v, c = d["k"].clone(), d["v"].clone(), d["centroids"].clone()
        sel = dp.sparse_indices.clone()
        out = torch.full_like(d["q"], float("nan"))
        ws = _workspace(dp, K, bos, eos) if split else None
        _cabi.sparse_layer_fused(d["q"], c, k, v, out, dp.dense_indptr, dp.sparse_indptr, dp.dense_indices, sel,
                                 dp.last_page_len, dp.S, P, K, bos, eos, dp.max_pages, scale, nk, nv, loc,
                                 workspace=ws)
        res.append((k, v, c, sel, out))
    for a, b in zip(*res):
        assert torch.equal(a.view(torch.int16) if a.dtype == torch.bfloat16 else a,
                           b.view(torch.int16) if b.dtype == torch.bfloat16 else b)
    assert not torch.isnan(res[1][4].float()).any()
    # and against the separate kernels
    d = to_dev(prob)
    k, v, c = d["k"].clone(), d["v"].clone(), d["centroids"].clone()
    sel = dp.sparse_indices.clone()
    out = torch.empty_like(d["q"])
    _cabi.set_kv_cmean(k, v, nk, nv, c, loc, P)
    _cabi.indexer_fused(d["q"], c, dp.dense_indptr, dp.sparse_indptr, dp.dense_indices, sel, dp.S, K, bos, eos,
                        dp.max_pages)
    _cabi.decode_gqa(d["q"], k, v, out, dp.sparse_indptr, sel, dp.last_page_len, dp.S, P, scale)
    assert torch.equal(sel, res[1][3])
    assert torch.equal(out.view(torch.int16), res[1][4].view(torch.int16))


def test_quest_layer_split_matches_unsplit():
    seq, H, G, D, P, K, bos, eos = [20000, 1000, 8300], 4, 4, 128, 16, 30, 1, 1
    prob = vo.make_paged_problem(47, seq, H, G, D, P)
    kf = prob["k"].float()
    cmax, cmin = kf.max(dim=1, keepdim=True).values.bfloat16(), kf.min(dim=1, keepdim=True).values.bfloat16()
    dp = DevicePlan(prob, P, H, K, bos, eos)
    ref = dp.oracle(prob)
    vo.forward_indexer_quest(prob["q"], cmax, cmin, ref, K, bos, eos)
    ns = int(ref["sparse_kv_indptr"][-1])
    d = to_dev(prob)
    outs = []
    for ws in (None, _workspace(dp, K, bos, eos)):
        sel = dp.sparse_indices.clone()
        out = torch.full_like(d["q"], float("nan"))
        _cabi.sparse_layer_fused(d["q"], cmax.cuda(), d["k"], d["v"], out, dp.dense_indptr, dp.sparse_indptr,
                                 dp.dense_indices, sel, dp.last_page_len, dp.S, P, K, bos, eos, dp.max_pages,
                                 1.0 / math.sqrt(D), quest_min=cmin.cuda(), workspace=ws)
        np.testing.assert_array_equal(sel.cpu().numpy()[:ns], ref["sparse_kv_indices"])
        outs.append(out)
    assert torch.equal(outs[0].view(torch.int16), outs[1].view(torch.int16))


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_indexer_fused_above_2048_candidates(dtype):
    """40000 tokens = 2500 pages: past the register sort, the keys are sorted in shared memory."""
    seq, H, G, D, P, K, bos, eos = [40000, 700], 2, 2, 128, 16, 30, 1, 1
    prob = vo.make_paged_problem(53, seq, H, G, D, P, dtype=dtype)
    dp = DevicePlan(prob, P, H, K, bos, eos)
    ref = dp.oracle(prob)
    vo.forward_indexer(prob["q"], prob["centroids"], ref, K, bos, eos)
    ns = int(ref["sparse_kv_indptr"][-1])
    d = to_dev(prob)
    sel = dp.sparse_indices.clone()
    _cabi.indexer_fused(d["q"], d["centroids"], dp.dense_indptr, dp.sparse_indptr, dp.dense_indices, sel, dp.S, K, bos,
                        eos, dp.max_pages)
    np.testing.assert_array_equal(sel.cpu().numpy()[:ns], ref["sparse_kv_indices"])
    if dtype == torch.bfloat16:  # the one-launch layer, unsplit (shared-memory sort) and split (5 chunks)
        for ws in (None, _workspace(dp, K, bos, eos)):
            sel = dp.sparse_indices.clone()
            out = torch.full_like(d["q"], float("nan"))
            _cabi.sparse_layer_fused(d["q"], d["centroids"], d["k"], d["v"], out, dp.dense_indptr, dp.sparse_indptr,
                                     dp.dense_indices, sel, dp.last_page_len, dp.S, P, K, bos, eos, dp.max_pages,
                                     1.0 / math.sqrt(D), workspace=ws)
            np.testing.assert_array_equal(sel.cpu().numpy()[:ns], ref["sparse_kv_indices"])
            want = vo.decode_gqa(prob["q"], prob["k"], prob["v"], ref["sparse_kv_indptr"], ref["sparse_kv_indices"],
                                 ref["kv_last_page_len"])
            assert close(out, want, BF16_TOL)


def test_understated_page_bound_raises_the_status_word():
    """max_num_pages_per_request below a request's real page count: the call still succeeds, the segment gets
    its first topk_val candidates (a well-defined list) and the sticky status word reports it."""
    seq, H, G, D, P, K, bos, eos = [8192, 300], 2, 2, 128, 16, 30, 1, 1
    prob, dp, ref = _problem(59, seq, H, G, D, P, K, bos, eos)
    d = to_dev(prob)
    assert _cabi.device_status(clear=True) == 0
    sel = dp.sparse_indices.clone()
    _cabi.indexer_fused(d["q"], d["centroids"], dp.dense_indptr, dp.sparse_indptr, dp.dense_indices, sel, dp.S, K, bos,
                        eos, 64)  # request 0 has 512 pages (the kernels always make room for 256 candidates)
    assert _cabi.device_status() & _cabi.STATUS_CANDIDATE_OVERFLOW
    got = sel.cpu().numpy()
    dip, sip, din = ref["dense_kv_indptr"], ref["sparse_kv_indptr"], ref["dense_kv_indices"]
    for s in range(H):  # request 0: first K candidates; request 1 (19 pages, copy path) untouched
        np.testing.assert_array_equal(got[sip[s] + bos: sip[s] + bos + K], din[dip[s] + bos: dip[s] + bos + K])
    assert _cabi.device_status(clear=True) & _cabi.STATUS_CANDIDATE_OVERFLOW
    assert _cabi.device_status() == 0
    # the same through the one-launch layer and the stand-alone top-k
    out = torch.empty_like(d["q"])
    _cabi.sparse_layer_fused(d["q"], d["centroids"], d["k"], d["v"], out, dp.dense_indptr, dp.sparse_indptr,
                             dp.dense_indices, sel, dp.last_page_len, dp.S, P, K, bos, eos, 64, 1.0 / math.sqrt(D))
    assert _cabi.device_status(clear=True) & _cabi.STATUS_CANDIDATE_OVERFLOW
    assert not torch.isnan(out.float()).any()
    scores = torch.zeros(int(dip[-1]), dtype=torch.bfloat16, device="cuda")
    _cabi.topk(scores, dp.dense_indptr, dp.sparse_indptr, dp.dense_indices, sel, dp.S, K, bos, eos, 64)
    assert _cabi.device_status(clear=True) & _cabi.STATUS_CANDIDATE_OVERFLOW
