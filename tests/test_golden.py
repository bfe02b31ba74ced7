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
