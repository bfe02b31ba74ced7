"""Stand-alone kernels of the chained indexer operators (GeMM, Softmax, Normalize, RAGGED reductions, binary
operators on BATCHED x PAGED and RAGGED x PAGED operands, Transpose, Save / Load) against the CPU oracle, bit
for bit, and user flows that compose them in ways the fused chains do not cover."""
import textwrap

import numpy as np
import pytest
import torch

from oracle import vortex_oracle as vo
from vortex_torch import _cabi

from _util import DevicePlan

pytestmark = pytest.mark.gpu


def _setup(seed, seq, H, G, D, P, K, bos=1, eos=1):
    prob = vo.make_paged_problem(seed, seq, H, G, D, P)
    dp = DevicePlan(prob, P, H, K, bos, eos)
    ref = dp.oracle(prob)
    win = (ref["dense_kv_indptr"], dp.S, K, bos, eos)
    dwin = (dp.dense_indptr, dp.S, K, bos, eos)
    mask = torch.zeros(int(ref["dense_kv_indptr"][-1]), dtype=torch.bool)
    for _, a, b in vo.candidate_windows(*win):
        mask[a:b] = True
    return prob, dp, ref, win, dwin, mask


def _same(got: torch.Tensor, want: torch.Tensor, mask) -> bool:
    n = mask.numel()
    return torch.equal(got.cpu()[:n][mask].view(torch.int16), want[:n][mask].view(torch.int16))


CASES = [([1024, 5000, 333, 17, 40], 4, 4, 128, 16, 8), ([700, 130], 2, 8, 64, 8, 5), ([3000], 2, 1, 128, 16, 30)]


@pytest.mark.parametrize("seq,H,G,D,P,K", CASES)
def test_gemm_softmax_max_stand_alone_equal_oracle_and_fused(seq, H, G, D, P, K):
    prob, dp, ref, win, dwin, mask = _setup(81, seq, H, G, D, P, K)
    n = mask.numel()
    q, cent = prob["q"].cuda(), prob["centroids"].cuda()
    mm = torch.full((n, 1, G), 7.0, dtype=torch.bfloat16, device="cuda")
    _cabi.gemm_bpr(q, cent, mm, dp.dense_indptr, dp.dense_indices, dp.S, K, 1, 1)
    want_mm = vo.gemm_bpr(prob["q"], prob["centroids"], ref["dense_kv_indptr"], ref["dense_kv_indices"], dp.S, K, 1, 1)
    assert _same(mm, want_mm, mask)
    assert bool((mm.cpu()[~mask] == 7.0).all())            # rows outside the candidate windows are not touched
    _cabi.softmax_ragged(mm, *dwin, 0.09)
    want_sm = vo.softmax_ragged(want_mm.clone(), *win, 0.09)
    assert _same(mm, want_sm, mask)
    red = torch.zeros(n, 1, 1, dtype=torch.bfloat16, device="cuda")
    _cabi.reduce_ragged(mm, red, 2, vo.REDUCE_MAX, *dwin)
    want = vo.reduce_ragged(want_sm, 2, vo.REDUCE_MAX, *win)
    assert _same(red, want, mask)
    # the three stand-alone kernels followed by the stand-alone top-k select what the fused chain selects
    sel_a, sel_b = dp.sparse_indices.clone(), dp.sparse_indices.clone()
    _cabi.topk(red.view(-1), dp.dense_indptr, dp.sparse_indptr, dp.dense_indices, sel_a, dp.S, K, 1, 1, dp.max_pages)
    _cabi.indexer_gqa_softmax_fused(q, cent, dp.dense_indptr, dp.sparse_indptr, dp.dense_indices, sel_b, dp.S, K, 1, 1,
                                    dp.max_pages, 0.09)
    assert torch.equal(sel_a, sel_b)


@pytest.mark.parametrize("kind", [vo.REDUCE_MEAN, vo.REDUCE_MAX, vo.REDUCE_MIN, vo.REDUCE_L2NORM, vo.REDUCE_SUM])
@pytest.mark.parametrize("dim", [1, 2])
@pytest.mark.parametrize("R,C", [(4, 128), (3, 20), (1, 1), (8, 300)])
def test_ragged_reductions_equal_oracle(kind, dim, R, C):
    seq, H, P, K = [900, 130, 40], 2, 8, 5
    prob, dp, ref, win, dwin, mask = _setup(83, seq, H, 1, 8, P, K)
    n = mask.numel()
    g = torch.Generator().manual_seed(R * 1000 + C)
    x = torch.randn(n, R, C, generator=g).bfloat16()
    out = torch.zeros((n, 1, C) if dim == 1 else (n, R, 1), dtype=torch.bfloat16, device="cuda")
    _cabi.reduce_ragged(x.cuda(), out, dim, kind, *dwin)
    assert _same(out, vo.reduce_ragged(x, dim, kind, *win), mask)


def test_normalize_equals_oracle():
    seq, H, P, K = [5000, 900, 40], 2, 8, 5
    prob, dp, ref, win, dwin, mask = _setup(85, seq, H, 1, 8, P, K)
    n = mask.numel()
    x = torch.randn(n, 2, 3, generator=torch.Generator().manual_seed(1)).bfloat16()
    xd = x.cuda()
    _cabi.normalize_ragged(xd, *dwin)
    assert _same(xd, vo.normalize_ragged(x.clone(), *win), mask)
    assert torch.equal(xd.cpu()[~mask], x[~mask])


@pytest.mark.parametrize("op,alpha,beta", [(vo.BINARY_MAX, 1, 1), (vo.BINARY_MIN, 1, 1), (vo.BINARY_ADD, 0.37, -2.5),
                                           (vo.BINARY_MUL, 1, 1)])
@pytest.mark.parametrize("seq,H,G,D,P,K", CASES[:2])
def test_binary_on_paged_operand_equals_oracle(op, alpha, beta, seq, H, G, D, P, K):
    prob, dp, ref, win, dwin, mask = _setup(87, seq, H, G, D, P, K)
    n = mask.numel()
    q, cent = prob["q"].cuda(), prob["centroids"].cuda()
    out = torch.zeros(n, G, D, dtype=torch.bfloat16, device="cuda")
    _cabi.binary_bpr(q, cent, out, dp.dense_indptr, dp.dense_indices, dp.S, K, 1, 1, op, alpha, beta)
    want = vo.binary_bpr(prob["q"], prob["centroids"], ref["dense_kv_indptr"], ref["dense_kv_indices"], dp.S, K, 1, 1,
                         op, alpha, beta)
    assert _same(out, want, mask)
    # RAGGED left operand: x[p] with table[row_p]
    x = torch.randn(n, G, 1, generator=torch.Generator().manual_seed(3)).bfloat16()
    out2 = torch.zeros(n, G, D, dtype=torch.bfloat16, device="cuda")
    _cabi.binary_bpr(x.cuda(), cent, out2, dp.dense_indptr, dp.dense_indices, dp.S, K, 1, 1, op, alpha, beta,
                     x_is_ragged=True)
    rows = torch.as_tensor(ref["dense_kv_indices"], dtype=torch.long)
    want2 = vo.elementwise_binary(x, prob["centroids"][rows], op, alpha, beta)
    assert _same(out2, want2, mask)


def test_quest_chain_from_stand_alone_kernels_equals_fused():
    seq, H, G, D, P, K = [2048, 1000, 333], 4, 2, 128, 16, 30
    prob, dp, ref, win, dwin, mask = _setup(89, seq, H, G, D, P, K)
    n = mask.numel()
    kf = prob["k"].float()
    cmax = kf.max(1, keepdim=True).values.bfloat16().cuda()
    cmin = kf.min(1, keepdim=True).values.bfloat16().cuda()
    q = prob["q"].cuda()
    hi = torch.zeros(n, G, D, dtype=torch.bfloat16, device="cuda")
    lo = torch.zeros_like(hi)
    _cabi.binary_bpr(q, cmax, hi, dp.dense_indptr, dp.dense_indices, dp.S, K, 1, 1, vo.BINARY_MUL)
    _cabi.binary_bpr(q, cmin, lo, dp.dense_indptr, dp.dense_indices, dp.S, K, 1, 1, vo.BINARY_MUL)
    u = torch.zeros_like(hi)
    _cabi.elementwise_binary(hi, lo, u, dp.dense_indptr[dp.S:dp.S + 1], vo.BINARY_MAX)
    s1 = torch.zeros(n, G, 1, dtype=torch.bfloat16, device="cuda")
    _cabi.reduce_ragged(u, s1, 2, vo.REDUCE_SUM, *dwin)
    s2 = torch.zeros(n, 1, 1, dtype=torch.bfloat16, device="cuda")
    _cabi.reduce_ragged(s1, s2, 1, vo.REDUCE_MAX, *dwin)
    want = vo.quest_scores(prob["q"], cmax.cpu(), cmin.cpu(), ref["dense_kv_indptr"], ref["dense_kv_indices"], dp.S, K,
                           1, 1)
    assert _same(s2.view(-1), want.view(-1), mask)
    sel_a, sel_b = dp.sparse_indices.clone(), dp.sparse_indices.clone()
    _cabi.topk(s2.view(-1), dp.dense_indptr, dp.sparse_indptr, dp.dense_indices, sel_a, dp.S, K, 1, 1, dp.max_pages)
    _cabi.indexer_quest_fused(q, cmax, cmin, dp.dense_indptr, dp.sparse_indptr, dp.dense_indices, sel_b, dp.S, K, 1, 1,
                              dp.max_pages)
    assert torch.equal(sel_a, sel_b)


def test_transpose_save_load():
    seq, H, P, K = [900, 130, 40], 2, 8, 5
    prob, dp, ref, win, dwin, mask = _setup(91, seq, H, 1, 8, P, K)
    n = mask.numel()
    x = torch.randn(n, 3, 5, generator=torch.Generator().manual_seed(2)).bfloat16()
    out = torch.zeros(n, 5, 3, dtype=torch.bfloat16, device="cuda")
    _cabi.transpose_ragged(x.cuda(), out, *dwin)
    assert _same(out, x.transpose(1, 2).contiguous(), mask)
    pool_rows = prob["centroids"].shape[0]
    paged = torch.zeros(pool_rows, 3, 5, dtype=torch.bfloat16, device="cuda")
    _cabi.save_load_ragged(x.cuda(), paged, dp.dense_indptr, dp.dense_indices, dp.S, K, 1, 1, save=True)
    rows = torch.as_tensor(ref["dense_kv_indices"], dtype=torch.long)
    want = torch.zeros(pool_rows, 3, 5, dtype=torch.bfloat16)
    want[rows[mask]] = x[mask]
    assert torch.equal(paged.cpu().view(torch.int16), want.view(torch.int16))
    back = torch.zeros(n, 3, 5, dtype=torch.bfloat16, device="cuda")
    _cabi.save_load_ragged(back, paged, dp.dense_indptr, dp.dense_indices, dp.S, K, 1, 1, save=False)
    assert _same(back, x, mask) and bool((back.cpu()[~mask] == 0).all())


# ------------------------------------------------------------------ compositions through the plugin API
def _run_indexer(flow, prob, seq, H, G, D, P, K):
    from test_gpu_flow import _runtime

    rt = _runtime(prob, seq, 1, H, G, D, P, K, 1, 1, torch.bfloat16, flow=flow, skip=())
    for name, t in rt.pool.buffers[0].items():
        if name in prob:
            t.copy_(prob[name])
    rt.plan(torch.as_tensor(prob["seq_lens"]).cuda(), torch.as_tensor(prob["req_indices"]).cuda())
    flow.forward_indexer(prob["q"].cuda(), rt.backend.kv_indices_decode[1].view(-1, 1, 1), rt.pool.buffers[0],
                         ctx=rt.ictx)
    torch.cuda.synchronize()
    return rt


FLOW_RELU = textwrap.dedent('''
    from vortex_torch.flow import vFlow, register
    from vortex_torch.indexer import GeMM, Softmax, Relu, Max, topK
    from vortex_torch.cache import Mean as CMean

    @register("probe_gemm_softmax_relu_max")
    class Probe(vFlow):
        def __init__(self):
            super().__init__()
            self.gemm, self.softmax, self.relu = GeMM(), Softmax(dim=0, scale=0.09), Relu(alpha=0.004, beta=0.0)
            self.max_op, self.output_func, self.reduction = Max(dim=2), topK(), CMean(dim=1)
        def forward_indexer(self, q, o, cache, ctx):
            score = self.gemm(q, cache["centroids"], ctx=ctx)
            self.softmax(score, ctx=ctx)
            kept = self.relu(score, ctx=ctx)
            self.output_func(self.max_op(kept, ctx=ctx), o, ctx=ctx)
        def forward_cache(self, cache, loc, ctx):
            self.reduction(cache["k"], cache["centroids"], loc=loc, ctx=ctx)
        def create_cache(self, page_size, head_dim):
            return {"centroids": (1, head_dim)}
''')


def test_user_flow_gemm_softmax_relu_max_topk(tmp_path):
    """A composition no fused chain covers: every operator runs its own kernel and the selection is the one the
    oracle's operators give."""
    from vortex_torch.flow import build_vflow

    f = tmp_path / "probe_relu_flow.py"
    f.write_text(FLOW_RELU)
    flow = build_vflow("probe_gemm_softmax_relu_max", {}, str(f))
    seq, H, G, D, P, K = [2048, 900, 300], 4, 4, 128, 16, 10
    prob = vo.make_paged_problem(93, seq, H, G, D, P)
    rt = _run_indexer(flow, prob, seq, H, G, D, P, K)
    assert flow.output_func._gqa_chain is None
    ref = vo.plan_decode(prob["seq_lens"], prob["req_to_token"], prob["req_indices"], P, H, K, 1, 1, 64, 16)
    S = prob["q"].shape[0]
    win = (ref["dense_kv_indptr"], S, K, 1, 1)
    mm = vo.gemm_bpr(prob["q"], prob["centroids"], ref["dense_kv_indptr"], ref["dense_kv_indices"], S, K, 1, 1)
    vo.softmax_ragged(mm, *win, 0.09)
    kept = vo.elementwise(mm, 0, 0.004, 0.0)
    scores = vo.reduce_ragged(kept, 2, vo.REDUCE_MAX, *win).view(-1)
    vo.topk_select(scores, ref["dense_kv_indptr"], ref["sparse_kv_indptr"], ref["dense_kv_indices"],
                   ref["sparse_kv_indices"], S, K, 1, 1)
    ns = int(ref["sparse_kv_indptr"][-1])
    np.testing.assert_array_equal(rt.backend.kv_indices_decode[1].cpu().numpy()[:ns], ref["sparse_kv_indices"])


FLOW_PEEK = textwrap.dedent('''
    from vortex_torch.flow import vFlow, register
    from vortex_torch.indexer import GeMM, Softmax, Max, L2Norm, topK
    from vortex_torch.cache import Mean as CMean

    @register("probe_gqa_with_a_second_reader")
    class Probe(vFlow):
        """The shipped gqa chain, whose softmax output a second operator also reads."""
        def __init__(self):
            super().__init__()
            self.gemm, self.softmax, self.max_op = GeMM(), Softmax(dim=0, scale=0.09), Max(dim=2)
            self.norm, self.output_func, self.reduction = L2Norm(dim=2), topK(), CMean(dim=1)
            self.seen = None
        def forward_indexer(self, q, o, cache, ctx):
            score = self.gemm(q, cache["centroids"], ctx=ctx)
            self.softmax(score, ctx=ctx)
            self.seen = self.norm(score, ctx=ctx)
            self.output_func(self.max_op(score, ctx=ctx), o, ctx=ctx)
        def forward_cache(self, cache, loc, ctx):
            self.reduction(cache["k"], cache["centroids"], loc=loc, ctx=ctx)
        def create_cache(self, page_size, head_dim):
            return {"centroids": (1, head_dim)}
''')


def test_chain_with_a_second_reader_runs_unfused_with_the_same_selection(tmp_path):
    from vortex_torch.flow import build_vflow

    f = tmp_path / "probe_peek_flow.py"
    f.write_text(FLOW_PEEK)
    flow = build_vflow("probe_gqa_with_a_second_reader", {}, str(f))
    seq, H, G, D, P, K = [2048, 900, 300], 4, 4, 128, 16, 10
    prob = vo.make_paged_problem(95, seq, H, G, D, P)
    rt = _run_indexer(flow, prob, seq, H, G, D, P, K)
    assert flow.output_func._gqa_chain is not None and not flow.output_func.chain_intact()
    ref = vo.plan_decode(prob["seq_lens"], prob["req_to_token"], prob["req_indices"], P, H, K, 1, 1, 64, 16)
    S = prob["q"].shape[0]
    vo.forward_indexer_gqa(prob["q"], prob["centroids"], ref, K, 1, 1, scale=0.09)
    ns = int(ref["sparse_kv_indptr"][-1])
    np.testing.assert_array_equal(rt.backend.kv_indices_decode[1].cpu().numpy()[:ns], ref["sparse_kv_indices"])
    # and the second reader saw the real softmax output
    win = (ref["dense_kv_indptr"], S, K, 1, 1)
    mm = vo.gemm_bpr(prob["q"], prob["centroids"], ref["dense_kv_indptr"], ref["dense_kv_indices"], S, K, 1, 1)
    vo.softmax_ragged(mm, *win, 0.09)
    want = vo.reduce_ragged(mm, 2, vo.REDUCE_L2NORM, *win)
    mask = torch.zeros(mm.shape[0], dtype=torch.bool)
    for _, a, b in vo.candidate_windows(*win):
        mask[a:b] = True
    assert _same(flow.seen, want, mask)
