"""Parity of the sm_100a kernels (called through the C ABI) against the CPU oracle.

Integer outputs (block tables, selected pages) and centroids must be bit-exact; attention outputs
must be within 2e-2 (abs or rel) for bf16 and 1e-5 for fp32.
"""
import math

import numpy as np
import pytest
import torch

from oracle import vortex_oracle as vo
from vortex_torch import _cabi

from _util import DevicePlan, assert_plan_equal, close, to_dev

pytestmark = pytest.mark.gpu
BF16_TOL, F32_TOL = 2e-2, 1e-5


# ------------------------------------------------------------------ block tables
@pytest.mark.parametrize("tables", [False, True])
@pytest.mark.parametrize("case", [
    dict(seq=[9, 18], P=4, H=2, K=1, bos=1, eos=1, mc=2),
    dict(seq=[24], P=4, H=1, K=1, bos=1, eos=2, mc=4),
    dict(seq=[16], P=4, H=1, K=1, bos=1, eos=2, mc=4),
    dict(seq=[1, 2, 3, 4, 5, 600, 77, 16, 1023, 31], P=16, H=8, K=3, bos=0, eos=1, mc=8),
    dict(seq=[4096] * 3 + [17, 512, 513], P=16, H=4, K=30, bos=1, eos=1, mc=64),
    dict(seq=[300] * 300, P=16, H=2, K=5, bos=2, eos=2, mc=4),          # more than one scan tile of requests
])
def test_plan_decode_bit_exact(case, tables):
    prob = vo.make_paged_problem(3, case["seq"], case["H"], 1, 8, case["P"], dtype=torch.float32)
    # shuffle request slots so req_indices is exercised
    bs = len(case["seq"])
    order = np.random.default_rng(0).permutation(bs)
    r2t = np.zeros_like(prob["req_to_token"])
    r2t[order] = prob["req_to_token"]
    prob["req_to_token"], prob["req_indices"] = r2t, order.astype(np.int64)
    dp = DevicePlan(prob, case["P"], case["H"], case["K"], case["bos"], case["eos"], max_chunk=case["mc"],
                    min_chunk=1, tables=tables)
    assert_plan_equal(dp, dp.oracle(prob))


def test_plan_decode_rejects_bad_arguments():
    z = torch.zeros(4, dtype=torch.int32, device="cuda")
    r2t = torch.zeros(1, 4, dtype=torch.int32, device="cuda")
    ridx = torch.zeros(1, dtype=torch.int64, device="cuda")
    with pytest.raises(RuntimeError, match="invalid argument"):
        _cabi.plan_decode(z[:1], r2t, ridx, z, z, z, z, z, z, z, z, z, z, 4, 1, 1, 0, 0, 4, 1)  # eos must be >= 1
    with pytest.raises(TypeError):
        _cabi.plan_decode(z[:1].long(), r2t, ridx, z, z, z, z, z, z, z, z, z, z, 4, 1, 1, 0, 1, 4, 1)


# ------------------------------------------------------------------ cache side
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_set_kv_layout(dtype):
    P, H, D, pages = 16, 8, 128, 12
    g = torch.Generator().manual_seed(0)
    k = torch.zeros(pages * H, P, D, dtype=dtype)
    v = torch.zeros(pages * H, P, D, dtype=dtype)
    loc = torch.randperm(pages * P, generator=g)[:50]
    nk = torch.randn(50, H, D, generator=g).to(dtype)
    nv = torch.randn(50, H, D, generator=g).to(dtype)
    kd, vd = k.cuda(), v.cuda()
    _cabi.set_kv(kd, vd, nk.cuda(), nv.cuda(), loc.cuda(), P)
    vo.set_kv(k, v, nk, nv, loc, P)
    assert torch.equal(kd.cpu(), k) and torch.equal(vd.cpu(), v)


@pytest.mark.parametrize("dtype,P,H,D", [(torch.bfloat16, 16, 8, 128), (torch.float32, 16, 8, 128),
                                         (torch.bfloat16, 64, 1, 576), (torch.bfloat16, 4, 2, 64),
                                         (torch.bfloat16, 12, 3, 128)])
def test_cmean_bit_exact(dtype, P, H, D):
    pages = 40
    g = torch.Generator().manual_seed(1)
    x = torch.randn(pages * H, P, D, generator=g).to(dtype)
    out = torch.zeros(pages * H, 1, D, dtype=dtype)
    closing = torch.randperm(pages, generator=g)[:17] * P + (P - 1)
    others = torch.randperm(pages, generator=g)[:9] * P + (P // 2 - 1 if P > 2 else 0)
    loc = torch.cat([closing, others])[torch.randperm(26, generator=g)]
    od = out.cuda()
    _cabi.cmean(x.cuda(), od, loc.cuda(), H, P)
    vo.cmean(x, out, loc, P, H)
    assert torch.equal(od.cpu().view(torch.int16 if dtype == torch.bfloat16 else torch.int32),
                       out.view(torch.int16 if dtype == torch.bfloat16 else torch.int32))


@pytest.mark.parametrize("dtype,P,H,D", [(torch.bfloat16, 16, 8, 128), (torch.float32, 16, 2, 128),
                                         (torch.bfloat16, 64, 1, 576), (torch.bfloat16, 5, 3, 64)])
def test_set_kv_cmean_fused_equals_separate(dtype, P, H, D):
    pages, nnz = 30, 21
    g = torch.Generator().manual_seed(4)
    k = torch.randn(pages * H, P, D, generator=g).to(dtype)
    v = torch.randn(pages * H, P, D, generator=g).to(dtype)
    cent = torch.randn(pages * H, 1, D, generator=g).to(dtype)
    pg = torch.randperm(pages, generator=g)[:nnz]
    loc = pg * P + torch.where(torch.arange(nnz) % 2 == 0, torch.full((nnz,), P - 1), torch.randint(0, P - 1, (nnz,), generator=g))
    nk = torch.randn(nnz, H, D, generator=g).to(dtype)
    nv = torch.randn(nnz, H, D, generator=g).to(dtype)
    k1, v1, c1 = k.cuda(), v.cuda(), cent.cuda()
    _cabi.set_kv_cmean(k1, v1, nk.cuda(), nv.cuda(), c1, loc.cuda(), P)
    vo.set_kv(k, v, nk, nv, loc, P)
    vo.cmean(k, cent, loc, P, H)
    assert torch.equal(k1.cpu(), k) and torch.equal(v1.cpu(), v)
    it = torch.int16 if dtype == torch.bfloat16 else torch.int32
    assert torch.equal(c1.cpu().view(it), cent.view(it))


def test_cmean_prefill_shape():
    """Config 4b scaled down: every slot of a long request; only page-closing slots work."""
    P, H, D, pages = 16, 8, 128, 128
    g = torch.Generator().manual_seed(2)
    x = torch.randn(pages * H, P, D, generator=g).bfloat16()
    loc = torch.arange(pages * P - 5)  # last page left incomplete
    od = torch.zeros(pages * H, 1, D, dtype=torch.bfloat16, device="cuda")
    _cabi.cmean(x.cuda(), od, loc.cuda(), H, P)
    want = torch.zeros(pages * H, 1, D, dtype=torch.bfloat16)
    rows = torch.arange((pages - 1) * H)
    want[rows, 0] = vo.cmean_pages(x, rows)
    assert torch.equal(od.cpu().view(torch.int16), want.view(torch.int16))


# ------------------------------------------------------------------ indexer
def _indexer_case(seed, seq, H, G, D, P, K, bos, eos, dtype):
    prob = vo.make_paged_problem(seed, seq, H, G, D, P, dtype=dtype)
    dp = DevicePlan(prob, P, H, K, bos, eos)
    ref = dp.oracle(prob)
    scores_ref = vo.forward_indexer(prob["q"], prob["centroids"], ref, K, bos, eos)
    return prob, dp, ref, scores_ref


INDEXER_CASES = [
    # seq lens, H, G, D, P, K, bos, eos, dtype
    ([4096], 8, 2, 128, 16, 30, 1, 1, torch.float32),                       # config 1
    ([2048, 2048, 1000, 600], 8, 2, 128, 16, 30, 1, 1, torch.bfloat16),     # config 2 shape, small batch
    ([1024, 5000, 333, 16, 17, 2500], 8, 4, 128, 16, 64, 1, 1, torch.bfloat16),  # config 3 shape, ragged
    ([700, 130], 2, 4, 64, 8, 5, 0, 2, torch.bfloat16),
    ([4096, 1300], 1, 16, 576, 64, 32, 1, 1, torch.bfloat16),               # config 5 shape (latent rows)
    ([1500], 2, 2, 256, 16, 7, 2, 1, torch.float32),
]


@pytest.mark.parametrize("case", INDEXER_CASES, ids=lambda c: f"H{c[1]}G{c[2]}D{c[3]}P{c[4]}K{c[5]}-{str(c[8])[6:]}")
def test_indexer_fused_and_split_match_oracle(case):
    seq, H, G, D, P, K, bos, eos, dtype = case
    prob, dp, ref, scores_ref = _indexer_case(11, seq, H, G, D, P, K, bos, eos, dtype)
    d = to_dev(prob)
    ns = int(ref["sparse_kv_indptr"][-1])
    # fused
    sparse_fused = dp.sparse_indices.clone()
    _cabi.indexer_fused(d["q"], d["centroids"], dp.dense_indptr, dp.sparse_indptr, dp.dense_indices, sparse_fused,
                        dp.S, K, bos, eos, dp.max_pages)
    np.testing.assert_array_equal(sparse_fused.cpu().numpy()[:ns], ref["sparse_kv_indices"])
    # operator by operator: mean (oracle order) -> gemv -> topk
    qm = vo.q_group_mean(prob["q"]).cuda()
    scores = torch.zeros(max(1, int(ref["dense_kv_indptr"][-1])), dtype=dtype, device="cuda")
    _cabi.gemv(qm, d["centroids"], scores, dp.dense_indptr, dp.dense_indices, dp.S, K, bos, eos)
    itype = torch.int16 if dtype == torch.bfloat16 else torch.int32
    assert torch.equal(scores.cpu().view(itype), scores_ref.view(itype)), "GeMV scores differ in bits"
    sparse_split = dp.sparse_indices.clone()
    _cabi.topk(scores, dp.dense_indptr, dp.sparse_indptr, dp.dense_indices, sparse_split, dp.S, K, bos, eos,
               dp.max_pages)
    np.testing.assert_array_equal(sparse_split.cpu().numpy()[:ns], ref["sparse_kv_indices"])


@pytest.mark.parametrize("seq,H,G,D,P,K", [([2048, 1000, 600], 8, 2, 128, 16, 30), ([1024, 5000, 333, 17], 4, 4, 128, 16, 64),
                                           ([700, 130], 2, 8, 64, 8, 5), ([8192], 2, 1, 128, 16, 30)])
def test_indexer_gqa_softmax_fused_matches_oracle(seq, H, G, D, P, K):
    """gqa_block_sparse_attention indexer (GeMM -> Softmax -> Max -> topK): selection bit-exact."""
    bos, eos = 1, 1
    prob = vo.make_paged_problem(13, seq, H, G, D, P)
    dp = DevicePlan(prob, P, H, K, bos, eos)
    ref = dp.oracle(prob)
    vo.forward_indexer_gqa(prob["q"], prob["centroids"], ref, K, bos, eos, scale=0.09)
    d = to_dev(prob)
    sel = dp.sparse_indices.clone()
    _cabi.indexer_gqa_softmax_fused(d["q"], d["centroids"], dp.dense_indptr, dp.sparse_indptr, dp.dense_indices, sel,
                                    dp.S, K, bos, eos, dp.max_pages, 0.09)
    ns = int(ref["sparse_kv_indptr"][-1])
    np.testing.assert_array_equal(sel.cpu().numpy()[:ns], ref["sparse_kv_indices"])


def _envelopes(prob):
    k = prob["k"].float()
    return k.max(dim=1, keepdim=True).values.bfloat16(), k.min(dim=1, keepdim=True).values.bfloat16()


@pytest.mark.parametrize("seq,H,G,D,P,K", [([2048, 1000, 600], 8, 2, 128, 16, 30), ([1024, 5000, 333, 17], 4, 4, 128, 16, 64),
                                           ([700, 130], 2, 8, 64, 8, 5)])
def test_indexer_quest_fused_matches_oracle(seq, H, G, D, P, K):
    """gqa_quest_sparse_attention indexer (Multiply x2 -> Maximum -> Sum -> Max -> topK): selection bit-exact."""
    bos, eos = 1, 1
    prob = vo.make_paged_problem(14, seq, H, G, D, P)
    cmax, cmin = _envelopes(prob)
    dp = DevicePlan(prob, P, H, K, bos, eos)
    ref = dp.oracle(prob)
    vo.forward_indexer_quest(prob["q"], cmax, cmin, ref, K, bos, eos)
    sel = dp.sparse_indices.clone()
    _cabi.indexer_quest_fused(prob["q"].cuda(), cmax.cuda(), cmin.cuda(), dp.dense_indptr, dp.sparse_indptr,
                              dp.dense_indices, sel, dp.S, K, bos, eos, dp.max_pages)
    ns = int(ref["sparse_kv_indptr"][-1])
    np.testing.assert_array_equal(sel.cpu().numpy()[:ns], ref["sparse_kv_indices"])


@pytest.mark.parametrize("op", ["max", "min"])
@pytest.mark.parametrize("dtype,P,H,D", [(torch.bfloat16, 16, 8, 128), (torch.float32, 12, 3, 64)])
def test_cminmax_exact(op, dtype, P, H, D):
    pages = 40
    g = torch.Generator().manual_seed(6)
    x = torch.randn(pages * H, P, D, generator=g).to(dtype)
    out = torch.zeros(pages * H, 1, D, dtype=dtype)
    loc = torch.cat([torch.randperm(pages, generator=g)[:15] * P + (P - 1), torch.randperm(pages, generator=g)[:7] * P])
    od = out.cuda()
    _cabi.creduce(x.cuda(), od, loc.cuda(), H, P, 1 if op == "max" else 2)
    vo.cminmax(x, out, loc, P, H, op)
    assert torch.equal(od.cpu(), out)


def test_topk_heavy_ties():
    """Scores drawn from four values: selection must follow candidate order inside each tie class."""
    H, K, bos, eos, P = 2, 30, 1, 1, 16
    prob = vo.make_paged_problem(5, [8192, 3000], H, 2, 128, P)
    dp = DevicePlan(prob, P, H, K, bos, eos)
    ref = dp.oracle(prob)
    g = torch.Generator().manual_seed(9)
    total = int(ref["dense_kv_indptr"][-1])
    scores = torch.tensor([-1.0, 0.0, -0.0, 2.5])[torch.randint(0, 4, (total,), generator=g)].bfloat16()
    vo.topk_select(scores, ref["dense_kv_indptr"], ref["sparse_kv_indptr"], ref["dense_kv_indices"],
                   ref["sparse_kv_indices"], dp.S, K, bos, eos)
    out = dp.sparse_indices.clone()
    _cabi.topk(scores.cuda(), dp.dense_indptr, dp.sparse_indptr, dp.dense_indices, out, dp.S, K, bos, eos,
               dp.max_pages)
    np.testing.assert_array_equal(out.cpu().numpy()[:int(ref["sparse_kv_indptr"][-1])], ref["sparse_kv_indices"])


# ------------------------------------------------------------------ decode attention
DECODE_CASES = [
    ([4096], 8, 2, 128, 16, 30, 1, 1, torch.float32),
    ([2048, 777, 100, 16, 15, 1], 8, 2, 128, 16, 30, 1, 1, torch.bfloat16),
    ([1024, 5000, 333], 8, 4, 128, 16, 64, 1, 1, torch.bfloat16),
    ([700, 130, 9], 2, 4, 64, 8, 5, 0, 2, torch.bfloat16),
    ([513, 64], 4, 1, 128, 32, 4, 1, 1, torch.bfloat16),
    ([300], 1, 8, 128, 16, 4, 1, 1, torch.bfloat16),
]


@pytest.mark.parametrize("case", DECODE_CASES, ids=lambda c: f"H{c[1]}G{c[2]}D{c[3]}P{c[4]}-{str(c[8])[6:]}")
@pytest.mark.parametrize("sparse", [True, False])
def test_decode_gqa_matches_oracle(case, sparse):
    seq, H, G, D, P, K, bos, eos, dtype = case
    prob, dp, ref, _ = _indexer_case(21, seq, H, G, D, P, K, bos, eos, dtype)
    d = to_dev(prob)
    key = "sparse" if sparse else "dense"
    indptr, indices = ref[f"{key}_kv_indptr"], ref[f"{key}_kv_indices"]
    want = vo.decode_gqa(prob["q"], prob["k"], prob["v"], indptr, indices, ref["kv_last_page_len"])
    out = torch.empty_like(d["q"])
    _cabi.decode_gqa(d["q"], d["k"], d["v"], out, torch.as_tensor(indptr).cuda(), torch.as_tensor(indices).cuda(),
                     dp.last_page_len, dp.S, P, 1.0 / math.sqrt(D))
    tol = BF16_TOL if dtype == torch.bfloat16 else F32_TOL
    assert close(out, want, tol), f"max err {(out.float().cpu() - want.float()).abs().max()}"


@pytest.mark.parametrize("case", [c for c in DECODE_CASES if c[8] == torch.bfloat16],
                         ids=lambda c: f"H{c[1]}G{c[2]}D{c[3]}P{c[4]}")
def test_sparse_layer_fused_equals_indexer_then_decode(case):
    """One launch (selection + attention) gives the selection of the oracle and the bits of the two-launch path."""
    seq, H, G, D, P, K, bos, eos, dtype = case
    prob, dp, ref, _ = _indexer_case(23, seq, H, G, D, P, K, bos, eos, dtype)
    d = to_dev(prob)
    ns = int(ref["sparse_kv_indptr"][-1])
    sel2 = dp.sparse_indices.clone()
    out2 = torch.empty_like(d["q"])
    _cabi.indexer_fused(d["q"], d["centroids"], dp.dense_indptr, dp.sparse_indptr, dp.dense_indices, sel2, dp.S, K,
                        bos, eos, dp.max_pages)
    _cabi.decode_gqa(d["q"], d["k"], d["v"], out2, dp.sparse_indptr, sel2, dp.last_page_len, dp.S, P,
                     1.0 / math.sqrt(D))
    sel1 = dp.sparse_indices.clone()
    out1 = torch.full_like(d["q"], float("nan"))
    _cabi.sparse_layer_fused(d["q"], d["centroids"], d["k"], d["v"], out1, dp.dense_indptr, dp.sparse_indptr,
                             dp.dense_indices, sel1, dp.last_page_len, dp.S, P, K, bos, eos, dp.max_pages,
                             1.0 / math.sqrt(D))
    np.testing.assert_array_equal(sel1.cpu().numpy()[:ns], ref["sparse_kv_indices"])
    assert torch.equal(sel1, sel2)
    assert torch.equal(out1.view(torch.int16), out2.view(torch.int16))


@pytest.mark.parametrize("seq", [[2048, 1024, 4096, 512], [2047, 1000, 33, 4096]])
def test_sparse_layer_fused_with_token_append(seq):
    """The one-launch layer that also writes the new token equals set_kv_cmean + indexer + decode."""
    H, G, D, P, K, bos, eos = 8, 2, 128, 16, 30, 1, 1
    prob, dp, ref, _ = _indexer_case(29, seq, H, G, D, P, K, bos, eos, torch.bfloat16)
    bs = len(seq)
    loc = torch.as_tensor([int(prob["req_to_token"][r, seq[r] - 1]) for r in range(bs)], dtype=torch.int64)
    g = torch.Generator().manual_seed(5)
    nk = torch.randn(bs, H, D, generator=g).bfloat16().cuda()
    nv = torch.randn(bs, H, D, generator=g).bfloat16().cuda()
    res = []
    for fused in (False, True):
        d = to_dev(prob)
        k, v, c = d["k"].clone(), d["v"].clone(), d["centroids"].clone()
        sel = dp.sparse_indices.clone()
        out = torch.full_like(d["q"], float("nan"))
        if fused:
            _cabi.sparse_layer_fused(d["q"], c, k, v, out, dp.dense_indptr, dp.sparse_indptr, dp.dense_indices, sel,
                                     dp.last_page_len, dp.S, P, K, bos, eos, dp.max_pages, 1.0 / math.sqrt(D),
                                     nk, nv, loc.cuda())
        else:
            _cabi.set_kv_cmean(k, v, nk, nv, c, loc.cuda(), P)
            _cabi.indexer_fused(d["q"], c, dp.dense_indptr, dp.sparse_indptr, dp.dense_indices, sel, dp.S, K, bos, eos,
                                dp.max_pages)
            _cabi.decode_gqa(d["q"], k, v, out, dp.sparse_indptr, sel, dp.last_page_len, dp.S, P, 1.0 / math.sqrt(D))
        res.append((k, v, c, sel, out))
    for a, b in zip(res[0], res[1]):
        assert torch.equal(a.view(torch.int16) if a.dtype == torch.bfloat16 else a,
                           b.view(torch.int16) if b.dtype == torch.bfloat16 else b)
    assert not torch.isnan(res[1][4].float()).any()


@pytest.mark.parametrize("case", [c for c in DECODE_CASES if c[8] == torch.bfloat16],
                         ids=lambda c: f"H{c[1]}G{c[2]}D{c[3]}P{c[4]}")
@pytest.mark.parametrize("splits", [2, 3, 8])
def test_decode_gqa_splitkv_matches_oracle(case, splits):
    """Split page lists (also with more splits than pages) merged through the caller's workspace."""
    seq, H, G, D, P, K, bos, eos, dtype = case
    prob, dp, ref, _ = _indexer_case(21, seq, H, G, D, P, K, bos, eos, dtype)
    d = to_dev(prob)
    ws = torch.full((_cabi.splitkv_workspace_bytes(dp.S, G, D, splits) // 4,), float("nan"), device="cuda")
    for key in ("sparse", "dense"):
        indptr, indices = ref[f"{key}_kv_indptr"], ref[f"{key}_kv_indices"]
        want = vo.decode_gqa(prob["q"], prob["k"], prob["v"], indptr, indices, ref["kv_last_page_len"])
        out = torch.empty_like(d["q"])
        _cabi.decode_gqa_splitkv(d["q"], d["k"], d["v"], out, torch.as_tensor(indptr).cuda(),
                                 torch.as_tensor(indices).cuda(), dp.last_page_len, dp.S, P, 1.0 / math.sqrt(D),
                                 splits, ws)
        assert close(out, want, BF16_TOL), f"max err {(out.float().cpu() - want.float()).abs().max()}"
    with pytest.raises(RuntimeError, match="invalid argument"):
        _cabi.decode_gqa_splitkv(d["q"], d["k"], d["v"], out, dp.sparse_indptr, dp.sparse_indices, dp.last_page_len,
                                 dp.S, P, 1.0, splits, ws[:8])


def test_decode_is_invariant_to_page_order():
    """Size-independent property: permuting the middle pages of a list changes nothing beyond fp32 re-association."""
    seq, H, G, D, P, K = [3000], 4, 2, 128, 16, 30
    prob, dp, ref, _ = _indexer_case(4, seq, H, G, D, P, K, 1, 1, torch.bfloat16)
    d = to_dev(prob)
    ind = torch.as_tensor(ref["sparse_kv_indices"]).clone()
    ptr = ref["sparse_kv_indptr"]
    shuffled = ind.clone()
    g = torch.Generator().manual_seed(0)
    for s in range(dp.S):
        a, b = int(ptr[s]) + 1, int(ptr[s + 1]) - 1
        shuffled[a:b] = ind[a:b][torch.randperm(b - a, generator=g)]
    outs = []
    for lst in (ind, shuffled):
        o = torch.empty_like(d["q"])
        _cabi.decode_gqa(d["q"], d["k"], d["v"], o, torch.as_tensor(ptr).cuda(), lst.cuda(), dp.last_page_len, dp.S, P,
                         1.0 / math.sqrt(D))
        outs.append(o)
    assert close(outs[0], outs[1], 1e-2)


# ------------------------------------------------------------------ MLA block-table decode
@pytest.mark.parametrize("seq,K", [([4096, 1300, 64, 65, 1, 700], 32), ([16384, 8000], 32), ([100, 3000], 5)])
def test_mla_block_table_decode(seq, K):
    """Config-5 shapes: 16 heads over a 576-dim latent, page 64; plan (table form) -> fused indexer -> decode."""
    H, G, D, P, bos, eos = 1, 16, 576, 64, 1, 1
    prob = vo.make_paged_problem(31, seq, H, G, D, P, v_dim=8)
    dp = DevicePlan(prob, P, H, K, bos, eos, tables=True)
    ref = dp.oracle(prob)
    vo.forward_indexer(prob["q"], prob["centroids"], ref, K, bos, eos)
    d = to_dev(prob)
    _cabi.indexer_fused(d["q"], d["centroids"], dp.dense_indptr, dp.sparse_indptr, dp.dense_indices,
                        dp.sparse_indices, dp.S, K, bos, eos, dp.max_pages, sparse_page_table=dp.tables[2])
    bs = len(seq)
    for s in range(bs):  # the table rows hold the same selection as the packed list
        n = int(ref["sparse_kv_indptr"][s + 1] - ref["sparse_kv_indptr"][s])
        np.testing.assert_array_equal(dp.tables[2][s, :n].cpu().numpy(), ref["sparse_page_table"][s, :n])
    scale = 1.0 / math.sqrt(192.0)
    for table, lens, rt, rl in ((dp.tables[2], dp.tables[3], ref["sparse_page_table"], ref["sparse_cache_seqlens"]),
                                (dp.tables[0], dp.tables[1], ref["dense_page_table"], ref["dense_cache_seqlens"])):
        want = vo.decode_mla(prob["q"], prob["k"], rt, rl, 512, scale)
        out = torch.empty(bs, G, 512, dtype=torch.bfloat16, device="cuda")
        _cabi.decode_mla(d["q"], d["k"], out, table, lens, P, scale)
        assert close(out, want, BF16_TOL), f"max err {(out.float().cpu() - want.float()).abs().max()}"


@pytest.mark.parametrize("path", [0, 1])
@pytest.mark.parametrize("P", [16, 32, 64, 128, 256])
def test_mla_page_sizes_both_forms(P, path):
    """tcgen05 (path 0) and mma.sync (path 1) forms on every page size, ragged lengths incl. empty and
    one-token requests, full and partial last tiles; the cache rows past a request's end hold NaN."""
    g = torch.Generator().manual_seed(100 + P)
    seq = [0, 1, 127, 128, 129, 1000, 2048, 3 * P, 3 * P + 1, 5000]
    bs = len(seq)
    pages = [(n + P - 1) // P for n in seq]
    total = sum(pages) + 3
    perm = torch.randperm(total, generator=g).to(torch.int32)
    stride = max(pages) + 2
    table = torch.full((bs, stride), -1, dtype=torch.int32)
    cache = torch.randn(total, P, 576, generator=g).to(torch.bfloat16)
    at = 0
    for b, n in enumerate(seq):
        table[b, :pages[b]] = perm[at:at + pages[b]]
        at += pages[b]
        if n % P:  # poison the unwritten tail of the last page
            cache[int(table[b, pages[b] - 1]), n % P:] = float("nan")
    cache[perm[at:]] = float("nan")  # pages no request owns
    q = torch.randn(bs, 16, 576, generator=g).to(torch.bfloat16)
    lens = torch.tensor(seq, dtype=torch.int32)
    scale = 1.0 / math.sqrt(192.0)
    want = vo.decode_mla(q, cache, table.clamp(min=0).numpy(), lens.numpy(), 512, scale)
    out = torch.full((bs, 16, 512), 7.0, dtype=torch.bfloat16, device="cuda")
    old = _cabi.set_mla_path(path)
    try:
        _cabi.decode_mla(q.cuda(), cache.cuda(), out, table.clamp(min=0).cuda(), lens.cuda(), P, scale)
        torch.cuda.synchronize()
    finally:
        _cabi.set_mla_path(old)
    assert _cabi.mla_fault_bits() == 0
    assert not torch.isnan(out.float()).any()
    assert close(out, want, BF16_TOL), f"max err {(out.float().cpu() - want.float()).abs().max()}"


@pytest.mark.parametrize("path", [0, 1])
@pytest.mark.parametrize("seq,K", [([4096, 1300, 64, 65, 1, 700, 16384], 32), ([100, 3000, 9000], 5),
                                    ([16384, 2100 * 4], 64), ([5000, 6000], 100)])
def test_mla_sparse_layer_one_launch_equals_two(seq, K, path):
    """vtx_mla_sparse_layer (the selection as the first phase of the tcgen05 decode kernel; two launches for the
    mma.sync form and for more than 64 selected pages) against vtx_indexer_fused + vtx_decode_mla: the same
    packed selection, the same page-table rows, the same output bits; selection also against the oracle."""
    H, G, D, P, bos, eos = 1, 16, 576, 64, 1, 1
    prob = vo.make_paged_problem(37, seq, H, G, D, P, v_dim=8)
    ref = None
    res = []
    scale = 1.0 / math.sqrt(192.0)
    old = _cabi.set_mla_path(path)
    try:
        for fused in (False, True, True):  # the fused form twice: its scratch is the ring the decode just used
            dp = DevicePlan(prob, P, H, K, bos, eos, tables=True)
            ref = ref or dp.oracle(prob)
            d = to_dev(prob)
            out = torch.full((len(seq), G, 512), float("nan"), dtype=torch.bfloat16, device="cuda")
            if fused:
                _cabi.mla_sparse_layer(d["q"], d["centroids"], d["k"], out, dp.dense_indptr, dp.sparse_indptr,
                                       dp.dense_indices, dp.sparse_indices, dp.tables[2], dp.tables[3], P, K, bos, eos,
                                       dp.max_pages, scale)
            else:
                _cabi.indexer_fused(d["q"], d["centroids"], dp.dense_indptr, dp.sparse_indptr, dp.dense_indices,
                                    dp.sparse_indices, dp.S, K, bos, eos, dp.max_pages, sparse_page_table=dp.tables[2])
                _cabi.decode_mla(d["q"], d["k"], out, dp.tables[2], dp.tables[3], P, scale)
            torch.cuda.synchronize()
            res.append((dp.sparse_indices.clone(), dp.tables[2].clone(), out))
    finally:
        _cabi.set_mla_path(old)
    assert _cabi.mla_fault_bits() == 0 and _cabi.device_status() == 0
    vo.forward_indexer(prob["q"], prob["centroids"], ref, K, bos, eos)
    ns = int(ref["sparse_kv_indptr"][-1])
    np.testing.assert_array_equal(res[0][0].cpu().numpy()[:ns], ref["sparse_kv_indices"])
    for other in res[1:]:
        assert torch.equal(other[0][:ns], res[0][0][:ns])
        for b in range(len(seq)):
            n = int(ref["sparse_kv_indptr"][b + 1] - ref["sparse_kv_indptr"][b])
            assert torch.equal(other[1][b, :n], res[0][1][b, :n])
        assert torch.equal(other[2].view(torch.int16), res[0][2].view(torch.int16))
    want = vo.decode_mla(prob["q"], prob["k"], ref["sparse_page_table"], ref["sparse_cache_seqlens"], 512, scale)
    assert close(res[1][2], want, BF16_TOL)


def test_mla_rejects_other_shapes():
    z = torch.zeros(1, 8, 576, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(RuntimeError, match="not supported"):
        _cabi.decode_mla(z, torch.zeros(1, 64, 576, dtype=torch.bfloat16, device="cuda"),
                         torch.zeros(1, 8, 512, dtype=torch.bfloat16, device="cuda"),
                         torch.zeros(1, 4, dtype=torch.int32, device="cuda"), torch.ones(1, dtype=torch.int32, device="cuda"),
                         64, 0.1)


def test_empty_batches_are_no_ops():
    """bs = 0 (or no new tokens): every entry point on the path returns OK and leaves its outputs untouched.
    (torch hands out null pointers for empty tensors and the C ABI refuses null pointers, so the Python wrappers
    return before the call; the planner's C entry point also accepts null per-request inputs at batch size 0.)"""
    P, H, G, D, K = 16, 2, 2, 128, 4
    i32 = dict(dtype=torch.int32, device="cuda")
    z = torch.zeros(8, **i32)
    canary = torch.full((8,), 77, **i32)
    q = torch.zeros(1, G, D, dtype=torch.bfloat16, device="cuda")[:0]
    kv = torch.zeros(4 * H, P, D, dtype=torch.bfloat16, device="cuda")
    cent = torch.zeros(4 * H, 1, D, dtype=torch.bfloat16, device="cuda")
    out = torch.zeros(1, G, D, dtype=torch.bfloat16, device="cuda")[:0]
    sel = canary.clone()
    _cabi.plan_decode(torch.zeros(1, **i32)[:0], torch.zeros(1, 64, **i32), torch.zeros(1, dtype=torch.int64, device="cuda")[:0],
                      z, z.clone(), z.clone(), sel, z.clone(), z.clone(), z.clone(), z.clone(), z[:1].clone(), z[:1].clone(),
                      P, H, K, 1, 1, 64, 16)
    _cabi.indexer_fused(q, cent, z, z, z, sel, 0, K, 1, 1, 8)
    _cabi.decode_gqa(q, kv, kv, out, z, z, z, 0, P, 0.1)
    _cabi.sparse_layer_fused(q, cent, kv, kv, out, z, z, z, sel, z, 0, P, K, 1, 1, 8, 0.1)
    empty_loc = torch.zeros(1, dtype=torch.int64, device="cuda")[:0]
    nk = torch.zeros(1, H, D, dtype=torch.bfloat16, device="cuda")[:0]
    before = kv.clone()
    _cabi.set_kv(kv, kv.clone(), nk, nk, empty_loc, P)
    _cabi.set_kv_cmean(kv, kv.clone(), nk, nk, cent, empty_loc, P)
    _cabi.cmean(kv, cent, empty_loc, H, P)
    torch.cuda.synchronize()
    assert torch.equal(sel, canary) and torch.equal(kv, before) and _cabi.device_status() == 0
