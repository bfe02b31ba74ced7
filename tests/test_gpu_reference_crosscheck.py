"""Cross-check against the reference project's own CUDA kernels (compiled for sm_100 into oracle/_ref).

The reference's native decode-path functions - the block-table planner and the top-k page selection -
are run on the same inputs as this repository's kernels and must agree bit for bit.  Skipped when the
cross-check extension was not built (it is built from the reference checkout by oracle/build_ref.py).
"""
import numpy as np
import pytest
import torch

from oracle import build_ref
from oracle import vortex_oracle as vo
from vortex_torch import _cabi

from _util import DevicePlan

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ref():
    mod = build_ref.load() if build_ref.built_module_path() is not None else None
    if mod is None:
        pytest.skip("oracle/_ref cross-check extension not built")
    return mod


CASES = [
    dict(seq=[9, 18, 40, 64], P=4, H=2, K=1, bos=1, eos=1, mc=2),
    dict(seq=[24, 16, 100], P=4, H=1, K=1, bos=1, eos=2, mc=4),
    dict(seq=[1, 2, 3, 4, 5, 600, 77, 16, 1023, 31], P=16, H=8, K=3, bos=0, eos=1, mc=8),
    dict(seq=[4096] * 3 + [17, 512, 513, 8192], P=16, H=4, K=30, bos=1, eos=1, mc=64),
    dict(seq=[300 + 7 * i for i in range(200)], P=16, H=2, K=5, bos=2, eos=2, mc=4),
]


def _ref_plan(ref, prob, c, tables):
    dev = "cuda"
    seq = torch.as_tensor(prob["seq_lens"], dtype=torch.int32, device=dev)
    r2t = torch.as_tensor(prob["req_to_token"], dtype=torch.int32, device=dev)
    ridx = torch.as_tensor(prob["req_indices"], dtype=torch.int64, device=dev)
    n = (np.asarray(prob["seq_lens"], dtype=np.int64) + c["P"] - 1) // c["P"]
    S = len(c["seq"]) * c["H"]
    budget = c["K"] + c["bos"] + c["eos"]
    i32 = dict(dtype=torch.int32, device=dev)
    out = dict(dip=torch.full((S + 1,), -1, **i32), din=torch.full((int(n.sum()) * c["H"],), -1, **i32),
               sip=torch.full((S + 1,), -1, **i32), sin=torch.full((int(np.minimum(n, budget).sum()) * c["H"],), -1, **i32),
               last=torch.full((S,), -1, **i32))
    nw = int(n.sum()) * c["H"] + S
    w = [torch.full((nw,), -1, **i32) for _ in range(3)] + [torch.full((1,), -1, **i32), torch.full((1,), -1, **i32)]
    out["w"] = w
    if tables:
        stride = int(n.max()) + 3
        out["t"] = [torch.full((S, stride), -1, **i32), torch.full((S,), -1, **i32),
                    torch.full((S, stride), -1, **i32), torch.full((S,), -1, **i32)]
        ref.sglang_plan_decode_fa3(seq, out["dip"], out["din"], out["sip"], out["sin"], out["t"][0], out["t"][1],
                                   out["t"][2], out["t"][3], r2t, ridx, *w, c["P"], c["H"], c["K"], c["bos"],
                                   c["eos"], c["mc"], 1)
    else:
        ref.sglang_plan_decode(seq, out["dip"], out["din"], out["sip"], out["sin"], out["last"], r2t, ridx, *w,
                               c["P"], c["H"], c["K"], c["bos"], c["eos"], c["mc"], 1)
    torch.cuda.synchronize()
    return out


@pytest.mark.parametrize("tables", [False, True])
@pytest.mark.parametrize("c", CASES, ids=lambda c: f"bs{len(c['seq'])}P{c['P']}H{c['H']}K{c['K']}")
def test_planner_equals_reference_kernels(ref, c, tables):
    prob = vo.make_paged_problem(5, c["seq"], c["H"], 1, 8, c["P"], dtype=torch.float32)
    mine = DevicePlan(prob, c["P"], c["H"], c["K"], c["bos"], c["eos"], max_chunk=c["mc"], min_chunk=1, tables=tables)
    r = _ref_plan(ref, prob, c, tables)
    eq = lambda a, b: torch.equal(a[: b.numel()].cpu(), b.cpu())
    assert eq(mine.dense_indptr, r["dip"]) and eq(mine.sparse_indptr, r["sip"])
    assert eq(mine.dense_indices, r["din"]) and eq(mine.sparse_indices, r["sin"])
    if not tables:
        assert eq(mine.last_page_len, r["last"])
    nw = int(r["w"][3].item())
    assert int(mine.w_num.item()) == nw and int(mine.w_chunk.item()) == int(r["w"][4].item())
    for a, b in ((mine.w_q, r["w"][0]), (mine.w_off, r["w"][1]), (mine.w_len, r["w"][2])):
        assert torch.equal(a[:nw].cpu(), b[:nw].cpu())
    if tables:
        for a, b in zip(mine.tables, r["t"]):
            assert torch.equal(a.cpu(), b.cpu())


@pytest.mark.parametrize("seq,H,K,bos,eos", [([8192, 3000, 600], 8, 30, 1, 1), ([4096, 100, 2000], 2, 64, 1, 2),
                                             ([65536], 1, 30, 1, 1), ([1500, 1700], 4, 7, 0, 1)])
@pytest.mark.parametrize("ties", [False, True])
def test_topk_equals_reference_kernel(ref, seq, H, K, bos, eos, ties):
    P = 16
    prob = vo.make_paged_problem(8, seq, H, 2, 128, P)
    dp = DevicePlan(prob, P, H, K, bos, eos)
    total = int(dp.dense_indptr[dp.S].item())
    g = torch.Generator().manual_seed(3)
    if ties:
        scores = torch.tensor([-1.0, 0.0, -0.0, 2.5, 0.125])[torch.randint(0, 5, (total,), generator=g)]
    else:
        scores = torch.randn(total, generator=g) * 11.3
    scores = scores.bfloat16().cuda()
    mine, theirs = dp.sparse_indices.clone(), dp.sparse_indices.clone()
    _cabi.topk(scores, dp.dense_indptr, dp.sparse_indptr, dp.dense_indices, mine, dp.S, K, bos, eos, dp.max_pages)
    ref.topk_output(scores, dp.dense_indptr, dp.sparse_indptr, dp.dense_indices, theirs, dp.S, K, bos, eos,
                    dp.max_pages)
    torch.cuda.synchronize()
    assert torch.equal(mine, theirs)


def test_indexer_selection_equals_recorded_reference_run():
    """The fused indexer and the one-launch layer against what the reference's own kernels (mv_bpr_kernel under
    Triton on a B200, then topk_output) selected on the same seeded bf16 batch of the config-2 shape
    (tests/golden/ref_gpu_triton_kernels.npz): the same pages in the same order for every segment, and the
    stand-alone GeMV returns the reference's score bits."""
    from pathlib import Path

    from _util import to_dev

    g = np.load(Path(__file__).parent / "golden" / "ref_gpu_triton_kernels.npz")
    c = {k: int(g[k]) for k in ("seed", "H", "G", "D", "P", "K", "bos", "eos", "chunk")}
    seq = [int(x) for x in g["seq"]]
    prob = vo.make_paged_problem(c["seed"], seq, c["H"], c["G"], c["D"], c["P"])
    dp = DevicePlan(prob, c["P"], c["H"], c["K"], c["bos"], c["eos"], max_chunk=c["chunk"], min_chunk=16)
    d = to_dev(prob)
    ns = len(g["selected"])
    sel = dp.sparse_indices.clone()
    _cabi.indexer_fused(d["q"], d["centroids"], dp.dense_indptr, dp.sparse_indptr, dp.dense_indices, sel, dp.S,
                        c["K"], c["bos"], c["eos"], dp.max_pages)
    np.testing.assert_array_equal(sel.cpu().numpy()[:ns], g["selected"])
    sel2 = dp.sparse_indices.clone()
    out = torch.empty_like(d["q"])
    _cabi.sparse_layer_fused(d["q"], d["centroids"], d["k"], d["v"], out, dp.dense_indptr, dp.sparse_indptr,
                             dp.dense_indices, sel2, dp.last_page_len, dp.S, c["P"], c["K"], c["bos"], c["eos"],
                             dp.max_pages, 1.0 / np.sqrt(c["D"]))
    np.testing.assert_array_equal(sel2.cpu().numpy()[:ns], g["selected"])
    qm = vo.q_group_mean(prob["q"]).cuda()
    scores = torch.zeros(len(g["scores_bits"]), dtype=torch.bfloat16, device="cuda")
    _cabi.gemv(qm, d["centroids"], scores, dp.dense_indptr, dp.dense_indices, dp.S, c["K"], c["bos"], c["eos"])
    got = scores.view(torch.int16).cpu().numpy()
    ref_plan = dp.oracle(prob)
    for _, a, b in vo.candidate_windows(ref_plan["dense_kv_indptr"], dp.S, c["K"], c["bos"], c["eos"]):
        np.testing.assert_array_equal(got[a:b], g["scores_bits"][a:b])
