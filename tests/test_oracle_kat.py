"""Known-answer tests pinning the CPU oracle by hand-derived cases (no GPU, no reference import)."""
import math

import numpy as np
import torch

from oracle import vortex_oracle as vo


def _r2t_identity(bs, pages, P):
    """Request r's logical page j is physical page r*pages + j."""
    r2t = np.zeros((bs, pages * P), dtype=np.int32)
    for r in range(bs):
        r2t[r] = np.arange(pages * P) + r * pages * P
    return r2t


def test_plan_decode_hand_case():
    # P=4, H=2, K=1, bos=1, eos=1 -> budget 3.  Requests: 9 tokens (3 pages, copy path), 18 tokens (5 pages).
    P, H, K, bos, eos = 4, 2, 1, 1, 1
    r2t = _r2t_identity(2, 5, P)
    plan = vo.plan_decode([9, 18], r2t, [0, 1], P, H, K, bos, eos, max_chunk_size=2, min_chunk_size=1,
                          page_table_stride=6)
    assert plan["dense_kv_indptr"].tolist() == [0, 3, 6, 11, 16]
    assert plan["sparse_kv_indptr"].tolist() == [0, 3, 6, 9, 12]
    # request 0 pages 0,1,2 -> rows page*H + h
    assert plan["dense_kv_indices"][:6].tolist() == [0, 2, 4, 1, 3, 5]
    # request 1 physical pages 5..9
    assert plan["dense_kv_indices"][6:].tolist() == [10, 12, 14, 16, 18, 11, 13, 15, 17, 19]
    # copy path for request 0; request 1: bos page in slot 0, hole, last page in slot 2
    assert plan["sparse_kv_indices"].tolist() == [0, 2, 4, 1, 3, 5, 10, -1, 18, 11, -1, 19]
    assert plan["kv_last_page_len"].tolist() == [1, 1, 2, 2]
    # workloads: request 0 has 1 candidate (<= K: none); request 1 has 3 candidates -> 2 chunks per head
    assert plan["winfo_num_workloads"].tolist() == [4]
    assert plan["winfo_q_indices"].tolist() == [2, 2, 3, 3]
    assert plan["winfo_kv_offsets"].tolist() == [7, 9, 12, 14]
    assert plan["winfo_kv_lens"].tolist() == [2, 1, 2, 1]
    assert plan["winfo_chunk_size"].tolist() == [2]
    assert plan["dense_cache_seqlens"].tolist() == [9, 9, 18, 18]
    assert plan["sparse_cache_seqlens"].tolist() == [9, 9, 10, 10]  # min((3-1)*4 + 2, 18)
    assert plan["sparse_page_table"][2].tolist() == [10, -1, 18, -1, -1, -1]
    assert plan["dense_page_table"][3].tolist() == [11, 13, 15, 17, 19, -1]


def test_plan_decode_eos2_and_exact_page():
    # eos=2 as in the reference's example run; seq_len a multiple of P gives last_page_len == P.
    P, H, K, bos, eos = 4, 1, 1, 1, 2
    r2t = _r2t_identity(1, 6, P)
    plan = vo.plan_decode([24], r2t, [0], P, H, K, bos, eos, max_chunk_size=4)
    assert plan["kv_last_page_len"].tolist() == [4]
    assert plan["sparse_kv_indptr"].tolist() == [0, 4]
    assert plan["sparse_kv_indices"].tolist() == [0, -1, 4, 5]
    # exactly budget pages -> copy path
    plan = vo.plan_decode([16], r2t, [0], P, H, K, bos, eos, max_chunk_size=4)
    assert plan["sparse_kv_indices"].tolist() == [0, 1, 2, 3]
    assert plan["winfo_num_workloads"].tolist() == [0]


def test_topk_ties_and_order():
    # scores of 6 candidates behind one bos page; ties must keep ascending candidate order.
    dense_indptr = np.array([0, 8], dtype=np.int32)
    sparse_indptr = np.array([0, 5], dtype=np.int32)
    dense = np.array([100, 101, 102, 103, 104, 105, 106, 107], dtype=np.int32)
    sparse = np.full(5, -1, dtype=np.int32)
    scores = torch.tensor([9.0, 1.0, 3.0, 3.0, -2.0, 3.0, 0.5, 9.0], dtype=torch.bfloat16)
    vo.topk_select(scores, dense_indptr, sparse_indptr, dense, sparse, 1, 3, 1, 1)
    # candidates are positions 1..6 -> (3.0@2, 3.0@3, 3.0@5) win, in position order
    assert sparse.tolist() == [-1, 102, 103, 105, -1]
    # -0.0 ties with +0.0
    scores = torch.tensor([0.0, -1.0, -0.0, 0.0, -3.0, -2.0, -5.0, 0.0], dtype=torch.float32)
    sparse[:] = -1
    vo.topk_select(scores, dense_indptr, sparse_indptr, dense, sparse, 1, 3, 1, 1)
    assert sparse.tolist() == [-1, 102, 103, 101, -1]


def test_topk_skips_short_segments():
    dense_indptr = np.array([0, 5], dtype=np.int32)
    sparse_indptr = np.array([0, 5], dtype=np.int32)
    dense = np.arange(5, dtype=np.int32)
    sparse = np.arange(5, dtype=np.int32) + 50
    vo.topk_select(torch.zeros(5), dense_indptr, sparse_indptr, dense, sparse, 1, 3, 1, 1)  # 3 candidates <= K
    assert sparse.tolist() == [50, 51, 52, 53, 54]


def test_cmean_trigger_and_value():
    P, H, D = 4, 2, 8
    x = torch.arange(3 * H * P * D, dtype=torch.float32).reshape(3 * H, P, D).to(torch.bfloat16)
    out = torch.zeros(3 * H, 1, D, dtype=torch.bfloat16)
    vo.cmean(x, out, torch.tensor([3, 6, 11]), P, H)  # slots 3 and 11 close pages 0 and 2; 6 does not
    for pid in (0, 1, 4, 5):
        want = x[pid].float().sum(0) / P
        assert torch.equal(out[pid, 0], want.to(torch.bfloat16))
    assert out[2].abs().sum() == 0 and out[3].abs().sum() == 0


def test_canonical_dot_close_to_exact_and_order_sensitive_cases():
    g = torch.Generator().manual_seed(1)
    for D in (64, 128, 576):
        rows = torch.randn(33, D, generator=g).bfloat16().float()
        vec = torch.randn(D, generator=g).bfloat16().float()
        exact = (rows.double() * vec.double()).sum(1)
        got = vo.canonical_dot(rows, vec, bf16_products=False)
        assert torch.allclose(got.double(), exact, rtol=1e-5, atol=1e-4)
        got_b = vo.canonical_dot(rows, vec, bf16_products=True)
        assert torch.allclose(got_b.double(), exact, rtol=0, atol=0.25)
    # a case where the order is visible: 1 + 2^-24 terms
    D = 128
    rows = torch.zeros(1, D)
    rows[0, 0] = 1.0
    rows[0, 8:16] = 2.0 ** -24  # chunk 1 -> lane 1: its partial sum 2^-21 survives the fold
    got = vo.canonical_dot(rows, torch.ones(D), bf16_products=False)
    assert got.item() == 1.0 + 2.0 ** -21


def test_config1_cpu_plumbing_matches_plain_torch():
    """The CPU-plumbing configuration: one request, 16 q heads, 8 KV heads, D=128, fp32, 256 pages, top-30 + 1 + 1."""
    P, H, G, D, K, bos, eos = 16, 8, 2, 128, 30, 1, 1
    prob = vo.make_paged_problem(0, [4096], H, G, D, P, dtype=torch.float32, permute=True)
    plan = vo.plan_decode(prob["seq_lens"], prob["req_to_token"], prob["req_indices"], P, H, K, bos, eos, 64)
    vo.forward_indexer(prob["q"], prob["centroids"], plan, K, bos, eos)
    out = vo.decode_gqa(prob["q"], prob["k"], prob["v"], plan["sparse_kv_indptr"], plan["sparse_kv_indices"],
                        plan["kv_last_page_len"])
    assert out.shape == (8, 2, 128)
    perm = prob["perm"]
    for h in range(H):
        # independent restatement with stock torch ops
        kh = prob["k"][torch.as_tensor(perm[:256]) * H + h]            # [256, 16, 128] in logical order
        cent = kh.mean(1)
        qm = prob["q"][h].mean(0)
        sc = cent[1:255] @ qm
        top = torch.topk(sc, K).indices + 1
        sel = plan["sparse_kv_indices"][plan["sparse_kv_indptr"][h]:plan["sparse_kv_indptr"][h + 1]]
        logical = [int(np.where(perm[:256] * H + h == r)[0][0]) for r in sel]
        assert logical[0] == 0 and logical[-1] == 255
        assert sorted(logical[1:-1]) == sorted(top.tolist())
        # scores of the selected middle pages are in descending order
        mid = sc[torch.as_tensor(logical[1:-1]) - 1]
        assert bool((mid[:-1] >= mid[1:]).all())
        pages = torch.as_tensor(logical)
        kk = kh[pages].reshape(-1, D)
        vv = prob["v"][torch.as_tensor(perm[:256]) * H + h][pages].reshape(-1, D)
        ref = torch.softmax((prob["q"][h] @ kk.T) / math.sqrt(D), -1) @ vv
        assert torch.allclose(out[h], ref, atol=1e-5, rtol=1e-5)


def test_elementwise_known_answers():
    """Unary elementwise operators of the indexer: values that are exact in any arithmetic, plus the rounding
    points the oracle fixes (each bf16 operation rounds once)."""
    x = torch.tensor([-3.0, -0.5, 0.0, 0.25, 2.0]).bfloat16()
    assert vo.elementwise(x, 0, 0.0, 0.0).tolist() == [0.0, 0.0, 0.0, 0.25, 2.0]          # relu
    assert vo.elementwise(x, 0, 0.25, -1.0).tolist() == [-1.0, -1.0, -1.0, 0.25, 2.0]     # threshold / fill
    assert vo.elementwise(x, 3, 0.0, 1.0).tolist() == [3.0, 0.5, 0.0, 0.25, 2.0]           # abs
    assert vo.elementwise(x, 4, 1.0, 2.0).tolist() == [-5.0, 0.0, 1.0, 1.5, 5.0]           # 2x + 1, exact
    # 0.3 rounds to bf16 0.30078125; 0.30078125 * 2 = 0.6015625 exact; + 1.5 = 2.1015625 -> bf16 2.09375
    assert vo.elementwise(torch.tensor([2.0]).bfloat16(), 4, 1.5, 0.3).item() == 2.09375
    sig = vo.elementwise(x, 1, 0.0, -1.0).float()                                          # logistic sigmoid
    assert torch.allclose(sig, torch.sigmoid(x.float()), atol=4e-3)
    silu = vo.elementwise(x, 2, 0.0, -1.0).float()
    assert torch.allclose(silu, torch.nn.functional.silu(x.float()), atol=8e-3)
    big = torch.tensor([300.0, -300.0]).bfloat16()
    assert vo.elementwise(big, 1, 0.0, 1.0).tolist() == [0.0, 1.0]                         # exp overflow / underflow
