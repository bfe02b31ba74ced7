"""The CPU oracle against golden vectors recorded from the reference project's own CUDA kernels.

tests/golden/ref_cuda_kernels.npz was written by tests/golden/make_golden_ref_gpu.py on a B200 from the
reference's sglang_plan_decode, sglang_plan_decode_fa3 and topk_output (csrc/utils_sglang.cu,
csrc/topk.cu compiled for sm_100).  Every array the reference wrote must be reproduced bit for bit.
"""
from pathlib import Path

import numpy as np
import torch

from oracle import vortex_oracle as vo

GOLD = np.load(Path(__file__).parent / "golden" / "ref_cuda_kernels.npz")


def _cases():
    for ci in range(int(GOLD["n_cases"])):
        pre = f"c{ci}_"
        cfg = {k[len(pre) + 4:]: GOLD[k] for k in GOLD.files if k.startswith(pre + "cfg_")}
        yield pre, dict(seq=[int(x) for x in cfg["seq"]], P=int(cfg["P"]), H=int(cfg["H"]), K=int(cfg["K"]),
                        bos=int(cfg["bos"]), eos=int(cfg["eos"]), mc=int(cfg["mc"]))


def test_plan_decode_matches_reference_kernels():
    names = ["dense_kv_indptr", "dense_kv_indices", "sparse_kv_indptr", "sparse_kv_indices", "kv_last_page_len",
             "winfo_q_indices", "winfo_kv_offsets", "winfo_kv_lens", "winfo_num_workloads", "winfo_chunk_size",
             "dense_page_table", "dense_cache_seqlens", "sparse_page_table", "sparse_cache_seqlens"]
    n = 0
    for pre, c in _cases():
        stride = GOLD[pre + "dense_page_table"].shape[1]
        plan = vo.plan_decode(c["seq"], GOLD[pre + "req_to_token"], GOLD[pre + "req_indices"], c["P"], c["H"], c["K"],
                              c["bos"], c["eos"], c["mc"], 1, page_table_stride=stride)
        for name in names:
            np.testing.assert_array_equal(plan[name], GOLD[pre + name], err_msg=f"{pre}{name}")
        n += 1
    assert n == 4


def test_topk_matches_reference_kernel():
    for pre, c in _cases():
        scores = torch.from_numpy(GOLD[pre + "scores_bf16_bits"].copy()).view(torch.bfloat16)
        sparse = GOLD[pre + "sparse_kv_indices"].copy()
        S = len(c["seq"]) * c["H"]
        vo.topk_select(scores, GOLD[pre + "dense_kv_indptr"], GOLD[pre + "sparse_kv_indptr"],
                       GOLD[pre + "dense_kv_indices"], sparse, S, c["K"], c["bos"], c["eos"])
        np.testing.assert_array_equal(sparse, GOLD[pre + "topk_selected"], err_msg=pre)


# --------------------------------------------------------------------------- reference Triton kernels (CPU interpreter)
TRI = np.load(Path(__file__).parent / "golden" / "ref_triton_kernels.npz")


def _within_one_bf16_ulp(a: torch.Tensor, b: torch.Tensor) -> bool:
    """a, b hold bf16-representable fp32 values; neighbours in bf16 differ by at most 2^-7 relative."""
    return bool(((a - b).abs() <= b.abs() * 2.0 ** -7 + 1e-30).all())


def test_set_kv_layout_matches_reference_triton_kernel():
    H, P = int(TRI["H"]), int(TRI["P"])
    k = torch.zeros(TRI["setkv_k"].shape)
    v = torch.zeros(TRI["setkv_v"].shape)
    vo.set_kv(k, v, torch.from_numpy(TRI["setkv_new_k"]), torch.from_numpy(TRI["setkv_new_v"]),
              torch.from_numpy(TRI["setkv_loc"]), P)
    assert torch.equal(k, torch.from_numpy(TRI["setkv_k"])) and torch.equal(v, torch.from_numpy(TRI["setkv_v"]))


def test_cmean_matches_reference_triton_kernel_within_one_ulp():
    H, P = int(TRI["H"]), int(TRI["P"])
    k = torch.from_numpy(TRI["k"]).bfloat16()            # values are bf16-representable: exact
    out = torch.zeros(k.shape[0], 1, k.shape[2], dtype=torch.bfloat16)
    vo.cmean(k, out, torch.from_numpy(TRI["cmean_loc"]), P, H)
    want = torch.from_numpy(TRI["cmean_out"])
    touched = want.abs().sum(dim=(1, 2)) > 0
    assert int(touched.sum()) == 5 * H                    # 5 of the 7 slots close a page
    assert bool((out.float()[~touched] == 0).all())       # same trigger: untouched rows stay untouched
    assert _within_one_bf16_ulp(out.float(), want)


def test_gemv_matches_reference_triton_kernel_within_one_ulp():
    cents = torch.from_numpy(TRI["mv_centroids"])[:, 0]
    x = torch.from_numpy(TRI["mv_x"])[:, 0]
    idx = torch.from_numpy(TRI["mv_indices"]).long()
    want = torch.from_numpy(TRI["mv_scores"]).view(-1)
    got = torch.zeros_like(want)
    for q, off, ln in zip(TRI["mv_wq"], TRI["mv_woff"], TRI["mv_wlen"]):
        rows = cents[idx[off:off + ln]]
        # the interpreter run used fp32 inputs: products are not rounded to bf16 there, only the score is
        got[off:off + ln] = vo.bf16_rne(vo.canonical_dot(rows, x[q], bf16_products=False))
    assert _within_one_bf16_ulp(got, want)
    # with bf16 products (what the kernels and the oracle use for bf16 inputs) the score moves by a few ulps at most
    for q, off, ln in zip(TRI["mv_wq"], TRI["mv_woff"], TRI["mv_wlen"]):
        rows = cents[idx[off:off + ln]]
        s = vo.bf16_rne(vo.canonical_dot(rows, x[q], bf16_products=True))
        assert bool(((s - want[off:off + ln]).abs() <= 0.25).all())


# --------------------------------------------------------------------------- operators of the two other shipped flows
# tests/golden/ref_triton_ops.npz: outputs of the reference's own Triton kernels (GeMM, Softmax, RAGGED
# reductions, elementwise binary, cache-side page reductions) under the Triton interpreter, made by
# tests/golden/make_golden_ref_triton_ops.py.  Maxima, minima and products must agree exactly, sums (whose
# order the interpreter takes from numpy) within one bf16 ulp.
OPS = np.load(Path(__file__).parent / "golden" / "ref_triton_ops.npz")


def _ops_layout():
    return OPS["indptr"], OPS["indices"], 3, int(OPS["topk"]), int(OPS["bos"]), int(OPS["eos"])


def _window_mask(total):
    indptr, _, eff, K, bos, eos = _ops_layout()
    m = torch.zeros(total, dtype=torch.bool)
    for _, a, b in vo.candidate_windows(indptr, eff, K, bos, eos):
        m[a:b] = True
    return m


def test_candidate_windows_are_the_reference_workloads():
    covered = np.zeros(int(OPS["indptr"][-1]), dtype=bool)
    for off, ln in zip(OPS["woff"], OPS["wlen"]):
        covered[off:off + ln] = True
    assert bool((torch.from_numpy(covered) == _window_mask(len(covered))).all())
    assert int(covered.sum()) == 12 + 298 + 7   # candidates of the 14-, 300- and 9-page segments (topk 4)


def _same_up_to_sum_order(got: torch.Tensor, want: torch.Tensor) -> bool:
    """The interpreter converts to bf16 by truncation; with the oracle asked to truncate too, the two differ
    only where the order of an fp32 sum moves the value across a bf16 boundary: never by more than one ulp
    and in under 1 % of the entries."""
    return _within_one_bf16_ulp(got, want) and float((got != want).float().mean()) < 0.01


def test_gemm_matches_reference_triton_kernel():
    indptr, indices, eff, K, bos, eos = _ops_layout()
    q, table = torch.from_numpy(OPS["q"]).bfloat16(), torch.from_numpy(OPS["table"]).bfloat16()
    want = torch.from_numpy(OPS["mm_out"])
    m = _window_mask(want.shape[0])
    got = vo.gemm_bpr(q, table, indptr, indices, eff, K, bos, eos, rounding="trunc").float()
    assert _same_up_to_sum_order(got[m], want[m])
    got = vo.gemm_bpr(q, table, indptr, indices, eff, K, bos, eos).float()   # the kernels' rounding
    assert _within_one_bf16_ulp(got[m], want[m])


def test_softmax_matches_reference_triton_kernel_within_one_ulp():
    """Input = the reference's own GeMM output, so that only the softmax is compared.  The 298-candidate
    segment exercises the reference's blocked accumulation (two blocks of 256 pages)."""
    indptr, _, eff, K, bos, eos = _ops_layout()
    want = torch.from_numpy(OPS["softmax_out"])
    m = _window_mask(want.shape[0])
    x = torch.from_numpy(OPS["mm_out"]).bfloat16()
    vo.softmax_ragged(x, indptr, eff, K, bos, eos, float(OPS["softmax_scale"]), rounding="trunc")
    assert _same_up_to_sum_order(x.float()[m], want[m])
    x = torch.from_numpy(OPS["mm_out"]).bfloat16()
    vo.softmax_ragged(x, indptr, eff, K, bos, eos, float(OPS["softmax_scale"]))
    assert _within_one_bf16_ulp(x.float()[m], want[m])
    assert torch.equal(x.float()[~m], torch.from_numpy(OPS["mm_out"])[~m])   # reserved pages untouched


def test_ragged_reductions_match_reference_triton_kernel():
    indptr, _, eff, K, bos, eos = _ops_layout()
    args = (indptr, eff, K, bos, eos)
    sm = torch.from_numpy(OPS["softmax_out"]).bfloat16()
    m = _window_mask(sm.shape[0])
    got = vo.reduce_ragged(sm, 2, vo.REDUCE_MAX, *args).float()
    assert torch.equal(got[m], torch.from_numpy(OPS["max_dim2_out"])[m])
    x = torch.from_numpy(OPS["reduce_in"]).bfloat16()
    kinds = dict(mean=vo.REDUCE_MEAN, max=vo.REDUCE_MAX, min=vo.REDUCE_MIN, l2norm=vo.REDUCE_L2NORM, sum=vo.REDUCE_SUM)
    for name, kind in kinds.items():
        for dim in (1, 2):
            got = vo.reduce_ragged(x, dim, kind, *args).float()
            want = torch.from_numpy(OPS[f"reduce_{name}_dim{dim}"])
            if name in ("max", "min"):
                assert torch.equal(got[m], want[m]), (name, dim)
            else:
                assert _within_one_bf16_ulp(got[m], want[m]), (name, dim)
                got = vo.reduce_ragged(x, dim, kind, *args, rounding="trunc").float()
                assert _same_up_to_sum_order(got[m], want[m]), (name, dim)


def test_binary_operators_match_reference_triton_kernel():
    indptr, indices, eff, K, bos, eos = _ops_layout()
    q, table = torch.from_numpy(OPS["q"]).bfloat16(), torch.from_numpy(OPS["table"]).bfloat16()
    rows = torch.from_numpy(OPS["bpr_rows"]).long()
    m = _window_mask(int(indptr[-1]))[rows]
    for name, op in (("mul", vo.BINARY_MUL), ("max", vo.BINARY_MAX), ("min", vo.BINARY_MIN)):
        got = vo.binary_bpr(q, table, indptr, indices, eff, K, bos, eos, op).float()[rows]
        # with fp32 stand-ins for bf16 inputs the reference kernel returns the unrounded product: round it once
        want = vo.bf16_rne(torch.from_numpy(OPS[f"bpr_{name}_out"]))
        assert torch.equal(got[m], want[m]), name
    a, b = torch.from_numpy(OPS["rrr_a"]).bfloat16(), torch.from_numpy(OPS["rrr_b"]).bfloat16()
    m = _window_mask(a.shape[0])
    for name, op in (("max", vo.BINARY_MAX), ("min", vo.BINARY_MIN)):
        got = vo.elementwise_binary(a, b, op).float()
        assert torch.equal(got[m], torch.from_numpy(OPS[f"rrr_{name}_out"])[m]), name
    # this kernel converts its product to bf16 itself, which the interpreter does by truncation
    exact = a.float() * b.float()
    assert torch.equal(vo.bf16_trunc(exact)[m], torch.from_numpy(OPS["rrr_mul_out"])[m])
    assert torch.equal(vo.elementwise_binary(a, b, vo.BINARY_MUL).float(), vo.bf16_rne(exact))


def test_cache_page_reductions_match_reference_triton_kernel():
    H, P = int(OPS["cache_H"]), int(OPS["cache_P"])
    k = torch.from_numpy(OPS["cache_k"]).bfloat16()
    loc = torch.from_numpy(OPS["cache_loc"])
    for op in ("max", "min"):
        out = torch.zeros(k.shape[0], 1, k.shape[2], dtype=torch.bfloat16)
        vo.cminmax(k, out, loc, P, H, op)
        assert torch.equal(out.float(), torch.from_numpy(OPS[f"cache_{op}_out"])), op
    out = torch.zeros(k.shape[0], 1, k.shape[2], dtype=torch.bfloat16)
    vo.cmean(k, out, loc, P, H)
    assert _within_one_bf16_ulp(out.float(), torch.from_numpy(OPS["cache_mean_out"]))


# --------------------------------------------------------------------------- the reference's kernels on a B200, bf16 inputs
# tests/golden/ref_gpu_triton_kernels.npz: what the reference's own mv_bpr_kernel (Triton, JIT-compiled for the
# B200), topk_output (csrc/topk.cu) and reduce_pp_kernel computed on a seeded bf16 batch of the config-2 shape,
# recorded by tests/golden/make_golden_ref_gpu_triton.py.  Inputs are regenerated from the seed.
REFGPU = np.load(Path(__file__).parent / "golden" / "ref_gpu_triton_kernels.npz")


def _refgpu_problem():
    c = {k: int(REFGPU[k]) for k in ("seed", "H", "G", "D", "P", "K", "bos", "eos", "chunk")}
    seq = [int(x) for x in REFGPU["seq"]]
    prob = vo.make_paged_problem(c["seed"], seq, c["H"], c["G"], c["D"], c["P"])
    plan = vo.plan_decode(prob["seq_lens"], prob["req_to_token"], prob["req_indices"], c["P"], c["H"], c["K"], c["bos"],
                          c["eos"], c["chunk"], 16)
    return c, seq, prob, plan


def test_scores_and_selection_equal_the_reference_kernels_on_bf16_inputs():
    """The canonical arithmetic of the oracle against the reference's real GPU kernels: the grouped-query
    mean, every one of the 10 984 candidate scores and all 32 selected page lists have the same bits."""
    c, seq, prob, plan = _refgpu_problem()
    S = len(seq) * c["H"]
    qm = vo.q_group_mean(prob["q"])
    assert np.array_equal(qm.view(torch.int16).numpy().reshape(-1), REFGPU["q_mean_bits"].reshape(-1))
    scores = vo.forward_indexer(prob["q"], prob["centroids"], plan, c["K"], c["bos"], c["eos"])
    want = REFGPU["scores_bits"]
    got = scores.view(torch.int16).numpy().reshape(-1)
    n = 0
    for _, a, b in vo.candidate_windows(plan["dense_kv_indptr"], S, c["K"], c["bos"], c["eos"]):
        np.testing.assert_array_equal(got[a:b], want[a:b])
        n += b - a
    assert n == 10984
    np.testing.assert_array_equal(plan["sparse_kv_indices"], REFGPU["selected"])


def test_cmean_deviation_from_the_reference_kernel_is_bounded():
    """The reference sums a page's rows in bf16 (cache/triton_kernels/reduce_impl.py:36-37); this build sums
    them in fp32 in row order and rounds once, as the benchmark's config 4 prescribes.  The two differ by
    rounding only: at most 2^-8 in absolute value on N(0,1) data."""
    c, seq, prob, plan = _refgpu_problem()
    rows = torch.from_numpy(REFGPU["cmean_rows"]).long()
    ref = torch.from_numpy(REFGPU["cmean_bits"].copy()).view(torch.bfloat16).float().view(len(rows), -1)
    got = vo.cmean_pages(prob["k"], rows).float().view(len(rows), -1)
    assert len(rows) == 4 * c["H"]          # four of the five slots close a page
    assert float((got - ref).abs().max()) <= 2.0 ** -8
    assert float((got == ref).float().mean()) > 0.4
