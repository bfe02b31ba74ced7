"""CPU oracle for the Vortex sparse-attention decode path (TEST INFRASTRUCTURE, not product).

This module restates, in PyTorch eager on CPU tensors, the arithmetic of the
reference's vFlow decode path: block-table planning, centroid maintenance,
the indexer (grouped-query mean, centroid GeMV, top-k page selection) and the
paged sparse decode attention.  Only the tests, the smoke check and the
CPU-baseline leg of the benchmark may import it; the product path never does.

Parity status
-------------
* Integer planning (`plan_decode`), top-k ordering and the KV layout follow the
  reference sources line by line (citations on each function).  They are pinned
  bit for bit by golden vectors recorded from the reference's own CUDA kernels
  (`sglang_plan_decode`, `sglang_plan_decode_fa3`, `topk_output`, compiled for
  sm_100 and run on a B200; tests/golden/ref_cuda_kernels.npz), by hand-derived
  known-answer cases, and on a GPU box by running those reference kernels side
  by side (tests/test_gpu_reference_crosscheck.py).
* Floating-point order: the reference's GeMV/CMean reduction order is whatever
  Triton's layout produced and is pinned by no reference test.  The oracle
  fixes one canonical order (documented on `canonical_dot`), and the CUDA
  kernels implement exactly that order, so selections are bit-exact between the
  two.  Against the reference's Triton kernels (run under the Triton
  interpreter, tests/golden/ref_triton_kernels.npz) the agreement is within one
  bf16 ulp, not bit-exact: **parity unpinned** for the reduction order.
* Paged attention and MLA decode are not in the reference tree at all (the
  attention lives in a third-party dependency, flashinfer-python 0.2.7.post1,
  called from an un-vendored SGLang fork; there is no MLA anywhere).  The oracle
  restates textbook softmax attention over the listed pages: **parity unpinned**.

All citations are paths inside the reference project.
"""
from __future__ import annotations

import math
from typing import Dict, Optional

import numpy as np
import torch

NEG_FILL = -1  # value used for "never written" integer slots in oracle outputs


# --------------------------------------------------------------------------- #
# numeric helpers
# --------------------------------------------------------------------------- #
def bf16_rne(x: torch.Tensor) -> torch.Tensor:
    """Round an fp32 tensor to bf16 (round-to-nearest-even) and return it as fp32."""
    return x.to(torch.float32).to(torch.bfloat16).to(torch.float32)


def bf16_trunc(x: torch.Tensor) -> torch.Tensor:
    """Truncate an fp32 tensor to bf16 (drop the low 16 bits) and return it as fp32.  Not a rounding any
    kernel uses: it is how the CPU interpreter of Triton converts to bf16, so the golden-vector tests ask for
    it when they compare with outputs recorded under that interpreter."""
    return (x.to(torch.float32).contiguous().view(torch.int32) & -65536).view(torch.float32)


def _round_bf16(x: torch.Tensor, rounding: str) -> torch.Tensor:
    """fp32 -> bf16 tensor with the named rounding ("rne": what the kernels do; "trunc": see `bf16_trunc`)."""
    assert rounding in ("rne", "trunc")
    return (bf16_trunc(x) if rounding == "trunc" else x.to(torch.float32)).to(torch.bfloat16)


def _pow2_ceil(n: int) -> int:
    p = 1
    while p < n:
        p *= 2
    return p


def canonical_lanes(head_dim: int) -> int:
    """Number of partial accumulators ("lanes") of the canonical dot product."""
    assert head_dim % 8 == 0, "head_dim must be a multiple of 8"
    return min(32, _pow2_ceil(head_dim // 8))


def canonical_dot(rows: torch.Tensor, vec: torch.Tensor, bf16_products: bool) -> torch.Tensor:
    """Dot product of every row of ``rows`` [R, D] with ``vec`` [D] in the canonical order.

    The reference computes ``sum((y_tile * x_i).to(float32), axis=1)`` where the
    product is formed in the input dtype (indexer/triton_kernels/mv_impl.py:60):
    for bf16 inputs each product is rounded to bf16 before the fp32 sum.  The
    order of that sum is not specified by the reference; this build fixes it:

    * the D dims are cut into chunks of 8 consecutive dims;
    * L = min(32, pow2ceil(D/8)) lanes; lane l owns chunks l, l+L, l+2L, ...
      and adds their products one at a time, in ascending dim order, into one
      fp32 accumulator that starts at +0.0 (separate multiply and add, no FMA);
    * the L lane sums are folded in halves: v[i] += v[i + w] for w = L/2 ... 1.

    ``rows`` and ``vec`` are fp32 tensors (bf16 values already widened).
    """
    R, D = rows.shape
    L = canonical_lanes(D)
    nch = D // 8
    prod = rows * vec.unsqueeze(0)                      # fp32 multiply, one rounding
    if bf16_products:
        prod = bf16_rne(prod)                           # exact product, RNE to bf16
    prod = prod.view(R, nch, 8)
    lane = torch.zeros(R, L, dtype=torch.float32)
    for c0 in range(0, nch, L):
        n = min(L, nch - c0)
        for j in range(8):
            lane[:, :n] = lane[:, :n] + prod[:, c0:c0 + n, j]
    w = L // 2
    while w >= 1:
        lane = lane[:, :w] + lane[:, w:2 * w]
        w //= 2
    return lane[:, 0]


# --------------------------------------------------------------------------- #
# KV layout and centroid maintenance
# --------------------------------------------------------------------------- #
def set_kv(k_cache, v_cache, new_k, new_v, loc, page_size: int) -> None:
    """Scatter new tokens into the paged caches.

    Follows cache/triton_kernels/set_kv.py:28-33: token slot ``t`` of head ``h``
    lives at flattened row ``(t // P) * H + h`` (caches are ``[num_pages*H, P, D]``)
    and token offset ``t % P``.
    """
    nnz, H, D = new_k.shape
    for i in range(nnz):
        t = int(loc[i])
        for h in range(H):
            row = (t // page_size) * H + h
            k_cache[row, t % page_size] = new_k[i, h]
            v_cache[row, t % page_size] = new_v[i, h]


def cmean(x: torch.Tensor, out: torch.Tensor, loc: torch.Tensor, page_size: int, num_kv_heads: int) -> None:
    """Page-completion mean over the token axis (the ``CMean(dim=1)`` cache op).

    Trigger and addressing follow cache/triton_kernels/reduce_impl.py:21-47: a new
    token at slot ``t`` does work only if ``(t + 1) % P == 0``; it then reduces the
    block ``x[(t // P) * H + h]`` of shape [rows, D] for every head h and writes
    ``out[(t // P) * H + h, 0, :]``.

    Arithmetic: fp32 accumulation over the rows in ascending order starting from
    +0.0, one division by the row count, one rounding to the cache dtype.  (The
    reference sums in bf16, reduce_impl.py:37; this build follows the fp32 rule.)
    """
    rows = x.shape[1]
    for t in loc.tolist():
        if (t + 1) % page_size != 0:
            continue
        for h in range(num_kv_heads):
            pid = (t // page_size) * num_kv_heads + h
            acc = torch.zeros(x.shape[2], dtype=torch.float32)
            blk = x[pid].to(torch.float32)
            for r in range(rows):
                acc = acc + blk[r]
            out[pid, 0] = (acc / float(rows)).to(out.dtype)


def cmean_pages(x: torch.Tensor, page_rows: torch.Tensor) -> torch.Tensor:
    """Vectorised form of the `cmean` arithmetic for many flattened rows at once (same order)."""
    blk = x[page_rows].to(torch.float32)
    acc = torch.zeros(blk.shape[0], blk.shape[2], dtype=torch.float32)
    for r in range(blk.shape[1]):
        acc = acc + blk[:, r]
    return (acc / float(blk.shape[1])).to(x.dtype)


# --------------------------------------------------------------------------- #
# block-table builder
# --------------------------------------------------------------------------- #
def plan_decode(
    cached_seq_lens,
    req_to_token,
    req_indices,
    page_size: int,
    num_kv_heads: int,
    topk_val: int,
    bos: int,
    eos: int,
    max_chunk_size: int,
    min_chunk_size: int = 1,
    page_table_stride: Optional[int] = None,
) -> Dict[str, np.ndarray]:
    """Block-table builder for one decode step.

    Restates csrc/utils_sglang.cu: indptr scan :257-309 (segments ordered
    (request, head); every head of a request has the same length), index fill
    :123-184 (dense row id ``(slot // P) * H + head``; sparse list = copy when
    pages <= budget, else BOS pages in front and EOS pages in the last slots,
    middle left for top-k), ``kv_last_page_len`` :148-151, workload chunks
    :188-254.  With ``page_table_stride`` set it also produces the block-table
    form of :949-1083 (page tables ``[bs*H, stride]`` and per-segment sequence
    lengths, sparse length ``min((budget-1)*P + last_len, seq_len)``).

    Slots the reference never writes hold ``NEG_FILL``.
    """
    seq = np.asarray(cached_seq_lens, dtype=np.int64)
    r2t = np.asarray(req_to_token, dtype=np.int64)
    ridx = np.asarray(req_indices, dtype=np.int64)
    bs = seq.shape[0]
    H, P, K = num_kv_heads, page_size, topk_val
    budget = K + bos + eos
    n = (seq + P - 1) // P
    m = np.minimum(budget, n)
    S = bs * H
    dense_indptr = np.zeros(S + 1, dtype=np.int32)
    sparse_indptr = np.zeros(S + 1, dtype=np.int32)
    cn = np.concatenate([[0], np.cumsum(n)])
    cm = np.concatenate([[0], np.cumsum(m)])
    for r in range(bs):
        for j in range(H + 1):
            dense_indptr[r * H + j] = H * cn[r] + j * n[r]
            sparse_indptr[r * H + j] = H * cm[r] + j * m[r]
    dense = np.full(int(dense_indptr[-1]), NEG_FILL, dtype=np.int32)
    sparse = np.full(int(sparse_indptr[-1]), NEG_FILL, dtype=np.int32)
    last = np.zeros(S, dtype=np.int32)
    out: Dict[str, np.ndarray] = {}
    if page_table_stride is not None:
        dpt = np.full((S, page_table_stride), NEG_FILL, dtype=np.int32)
        spt = np.full((S, page_table_stride), NEG_FILL, dtype=np.int32)
        dsl = np.zeros(S, dtype=np.int32)
        ssl = np.zeros(S, dtype=np.int32)
    for r in range(bs):
        toks = r2t[ridx[r]]
        nr = int(n[r])
        ll = int(seq[r] % P)
        ll = P if ll == 0 else ll
        for h in range(H):
            s = r * H + h
            last[s] = ll
            rows = (toks[np.arange(nr) * P] // P) * H + h
            d0 = dense_indptr[s]
            dense[d0:d0 + nr] = rows
            s0 = sparse_indptr[s]
            if nr <= budget:
                sparse[s0:s0 + nr] = rows
            else:
                sparse[s0:s0 + bos] = rows[:bos]
                for e in range(eos):
                    sparse[s0 + budget - e - 1] = rows[nr - e - 1]
            if page_table_stride is not None:
                dpt[s, :nr] = rows
                if nr <= budget:
                    spt[s, :nr] = rows
                else:
                    spt[s, :bos] = rows[:bos]
                    for e in range(eos):
                        spt[s, budget - e - 1] = rows[nr - e - 1]
                dsl[s] = seq[r]
                ssl[s] = min((budget - 1) * P + ll, int(seq[r]))
    # workload list (csrc/utils_sglang.cu:219-251)
    wq, woff, wlen = [], [], []
    for s in range(S):
        w = int(dense_indptr[s + 1] - dense_indptr[s]) - bos - eos
        cnt = w if w > K else 0
        nchunk = (cnt + max_chunk_size - 1) // max_chunk_size
        ll = cnt % max_chunk_size
        ll = max_chunk_size if ll == 0 else ll
        for j in range(nchunk):
            wq.append(s)
            wlen.append(max_chunk_size if j != nchunk - 1 else ll)
            woff.append(int(dense_indptr[s]) + j * max_chunk_size + bos)
    out.update(
        dense_kv_indptr=dense_indptr,
        sparse_kv_indptr=sparse_indptr,
        dense_kv_indices=dense,
        sparse_kv_indices=sparse,
        kv_last_page_len=last,
        winfo_q_indices=np.asarray(wq, dtype=np.int32),
        winfo_kv_offsets=np.asarray(woff, dtype=np.int32),
        winfo_kv_lens=np.asarray(wlen, dtype=np.int32),
        winfo_num_workloads=np.asarray([len(wq)], dtype=np.int32),
        winfo_chunk_size=np.asarray([max_chunk_size], dtype=np.int32),
    )
    if page_table_stride is not None:
        out.update(dense_page_table=dpt, sparse_page_table=spt,
                   dense_cache_seqlens=dsl, sparse_cache_seqlens=ssl)
    return out


# --------------------------------------------------------------------------- #
# indexer
# --------------------------------------------------------------------------- #
def q_group_mean(q: torch.Tensor) -> torch.Tensor:
    """Grouped-query mean ``q.mean(dim=1, keepdim=True)`` (flow/algorithms.py:168).

    fp32 accumulation over the group in ascending order from +0.0, one division
    by the group size, one rounding to q's dtype.
    """
    S, G, D = q.shape
    acc = torch.zeros(S, D, dtype=torch.float32)
    qf = q.to(torch.float32)
    for g in range(G):
        acc = acc + qf[:, g]
    return (acc / float(G)).to(q.dtype).view(S, 1, D)


def gemv_scores(q_mean, centroids, dense_indptr, dense_indices, eff_bs, topk_val, bos, eos,
                out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Centroid scores at packed dense positions (the ``GeMV`` indexer op).

    Follows indexer/triton_kernels/mv_impl.py:53-62 driven by the workload list of
    csrc/utils_sglang.cu:219-251: only the non-reserved candidates
    ``[indptr[s]+bos, indptr[s+1]-eos)`` of segments with more than ``topk_val``
    candidates are scored; the score of candidate position p is stored at
    ``out[p]`` in the input dtype.  Other positions are left untouched.
    """
    total = int(dense_indptr[eff_bs])
    dt = q_mean.dtype
    if out is None:
        out = torch.zeros(total, dtype=dt)
    is_bf16 = dt == torch.bfloat16
    cf = centroids.view(centroids.shape[0], -1)
    for s in range(eff_bs):
        a = int(dense_indptr[s]) + bos
        b = int(dense_indptr[s + 1]) - eos
        if b - a <= topk_val:
            continue
        rows = cf[torch.as_tensor(np.asarray(dense_indices[a:b]), dtype=torch.long)].to(torch.float32)
        sc = canonical_dot(rows, q_mean[s, 0].to(torch.float32), is_bf16)
        out.view(-1)[a:b] = sc.to(dt)
    return out


def _sortable(scores_f32: np.ndarray) -> np.ndarray:
    """Map fp32 values to uint32 keys whose unsigned order is the float order (-0.0 == +0.0)."""
    x = scores_f32.astype(np.float32) + np.float32(0.0)  # -0.0 + 0.0 = +0.0
    b = x.view(np.uint32)
    return np.where(b & 0x80000000, ~b, b | 0x80000000).astype(np.uint32)


def topk_select(scores, dense_indptr, sparse_indptr, dense_indices, sparse_indices,
                eff_bs, topk_val, bos, eos) -> None:
    """Top-k page selection (the ``topK`` indexer op), writing into ``sparse_indices``.

    Follows csrc/topk.cu:70-77, 97-112: candidates are the dense positions
    ``[indptr[s]+bos, indptr[s+1]-eos)``; segments with ``candidates <= topk_val``
    are skipped; keys are the scores widened to fp32, values the dense row ids;
    a stable descending sort (ties keep ascending candidate order) and the
    first ``topk_val`` values go to ``sparse[sparse_indptr[s] + bos + j]``.
    """
    sc = scores.detach().to(torch.float32).view(-1).numpy()
    for s in range(eff_bs):
        a = int(dense_indptr[s]) + bos
        b = int(dense_indptr[s + 1]) - eos
        if b - a <= topk_val:
            continue
        seg = sc[a:b]
        assert np.isfinite(seg).all(), "oracle defines ordering for finite scores only"
        keys = _sortable(seg).astype(np.int64)
        order = np.argsort(-keys, kind="stable")[:topk_val]
        o0 = int(sparse_indptr[s]) + bos
        sparse_indices[o0:o0 + topk_val] = np.asarray(dense_indices)[a + order]


def forward_indexer(q, centroids, plan, topk_val, bos, eos):
    """``q.mean -> GeMV -> topK`` of the block-sparse flow (flow/algorithms.py:168-170).

    ``plan`` is the dict returned by `plan_decode`; its ``sparse_kv_indices`` array
    is completed in place.  Returns the packed score tensor.
    """
    eff_bs = q.shape[0]
    qm = q_group_mean(q)
    scores = gemv_scores(qm, centroids, plan["dense_kv_indptr"], plan["dense_kv_indices"],
                         eff_bs, topk_val, bos, eos)
    topk_select(scores, plan["dense_kv_indptr"], plan["sparse_kv_indptr"], plan["dense_kv_indices"],
                plan["sparse_kv_indices"], eff_bs, topk_val, bos, eos)
    if "sparse_page_table" in plan:
        spt = plan["sparse_page_table"]
        for s in range(eff_bs):
            a, b = int(plan["sparse_kv_indptr"][s]), int(plan["sparse_kv_indptr"][s + 1])
            spt[s, : b - a] = plan["sparse_kv_indices"][a:b]
    return scores


# --------------------------------------------------------------------------- #
# decode attention
# --------------------------------------------------------------------------- #
def decode_gqa(q, k_cache, v_cache, indptr, indices, last_page_len, scale: Optional[float] = None):
    """Paged decode attention over each segment's page list.

    q ``[S, G, D]``; caches ``[num_pages*H, P, D]``; segment s attends to every
    token of the rows ``indices[indptr[s]:indptr[s+1]]`` except that the last
    listed row contributes only ``last_page_len[s]`` tokens (the data contract of
    csrc/utils_sglang.cu:148-151, 175-180).  fp32 softmax and accumulation,
    ``scale`` defaults to ``1/sqrt(D)``; output is rounded once to q's dtype.
    The attention kernel itself is third-party in the reference (flashinfer
    inside the SGLang fork): parity unpinned.
    """
    S, G, D = q.shape
    P = k_cache.shape[1]
    scale = 1.0 / math.sqrt(D) if scale is None else scale
    out = torch.zeros(S, G, v_cache.shape[2], dtype=torch.float32)
    for s in range(S):
        a, b = int(indptr[s]), int(indptr[s + 1])
        if b <= a:
            continue
        rows = torch.as_tensor(np.asarray(indices[a:b]), dtype=torch.long)
        ntok = (b - a - 1) * P + int(last_page_len[s])
        kk = k_cache[rows].to(torch.float32).reshape(-1, D)[:ntok]
        vv = v_cache[rows].to(torch.float32).reshape(-1, v_cache.shape[2])[:ntok]
        logits = (q[s].to(torch.float32) @ kk.T) * scale
        p = torch.softmax(logits, dim=-1)
        out[s] = p @ vv
    return out.to(q.dtype)


def decode_mla(q, latent_cache, page_table, cache_seqlens, kv_lora_rank: int, scale: float):
    """Block-table decode over a shared compressed latent (no counterpart in the reference).

    q ``[B, Hq, Dl]`` (Dl = kv_lora_rank + rope dims); ``latent_cache`` ``[pages, P, Dl]``;
    ``page_table`` ``[B, stride]`` row ids and ``cache_seqlens`` ``[B]`` token counts in the
    block-table form of csrc/utils_sglang.cu:968-976.  Keys are the full latent row,
    values its first ``kv_lora_rank`` dims.  fp32 softmax/accumulation, output
    ``[B, Hq, kv_lora_rank]`` rounded once to q's dtype.  Parity unpinned.
    """
    B, Hq, Dl = q.shape
    P = latent_cache.shape[1]
    out = torch.zeros(B, Hq, kv_lora_rank, dtype=torch.float32)
    for b in range(B):
        ntok = int(cache_seqlens[b])
        npg = (ntok + P - 1) // P
        rows = torch.as_tensor(np.asarray(page_table[b, :npg]), dtype=torch.long)
        kv = latent_cache[rows].to(torch.float32).reshape(-1, Dl)[:ntok]
        logits = (q[b].to(torch.float32) @ kv.T) * scale
        p = torch.softmax(logits, dim=-1)
        out[b] = p @ kv[:, :kv_lora_rank]
    return out.to(q.dtype)


# --------------------------------------------------------------------------- #
# seeded synthetic workload (shared by tests, smoke and the benchmark's CPU leg)
# --------------------------------------------------------------------------- #
def make_paged_problem(seed: int, seq_lens, num_kv_heads: int, group: int, head_dim: int,
                       page_size: int, dtype=torch.bfloat16, pool_pages: Optional[int] = None,
                       permute: bool = True, v_dim: Optional[int] = None):
    """Seeded paged-KV problem: N(0,1) q/K/V, random physical page order, centroids by `cmean_pages`."""
    g = torch.Generator().manual_seed(seed)
    seq = np.asarray(seq_lens, dtype=np.int32)
    bs = len(seq)
    n = (seq.astype(np.int64) + page_size - 1) // page_size
    max_pages = int(n.max())
    total = int(n.sum())
    pool_pages = total if pool_pages is None else pool_pages
    assert pool_pages >= total
    perm = torch.randperm(pool_pages, generator=g).numpy() if permute else np.arange(pool_pages)
    stride = max_pages * page_size
    r2t = np.zeros((bs, stride), dtype=np.int32)
    off = 0
    for r in range(bs):
        for j in range(int(n[r])):
            r2t[r, j * page_size:(j + 1) * page_size] = perm[off + j] * page_size + np.arange(page_size)
        off += int(n[r])
    H, D = num_kv_heads, head_dim
    vd = D if v_dim is None else v_dim
    k = torch.randn(pool_pages * H, page_size, D, generator=g).to(dtype)
    v = torch.randn(pool_pages * H, page_size, vd, generator=g).to(dtype)
    q = torch.randn(bs * H, group, D, generator=g).to(dtype)
    cent = torch.zeros(pool_pages * H, 1, D, dtype=dtype)
    full_rows = []
    off = 0
    for r in range(bs):
        nfull = int(seq[r]) // page_size
        for j in range(nfull):
            for h in range(H):
                full_rows.append(int(perm[off + j]) * H + h)
        off += int(n[r])
    if full_rows:
        fr = torch.as_tensor(full_rows, dtype=torch.long)
        cent[fr, 0] = cmean_pages(k, fr)
    return dict(seq_lens=seq, req_to_token=r2t, req_indices=np.arange(bs, dtype=np.int64),
                k=k, v=v, q=q, centroids=cent, perm=perm)


# --------------------------------------------------------------------------- #
# indexer of the gqa_block_sparse_attention flow
# --------------------------------------------------------------------------- #
def exp_canonical(x: np.ndarray) -> np.ndarray:
    """exp(x) for x <= 0 as a fixed sequence of fp32 operations (so CPU and GPU agree bit for bit).

    k = rint(x * log2(e)); r = x - k*ln2_hi - k*ln2_lo; degree-6 Taylor polynomial by Horner with separate
    multiplies and adds; result = p * 2^k.  Inputs below -87 give 0.  About 2 ulp from the true value.
    """
    f = np.float32
    x = np.asarray(x, dtype=f)
    k = np.rint(x * f(1.44269504)).astype(f)
    r = x - k * f(0.693145751953125)
    r = r - k * f(1.42860677e-6)
    p = f(1.0 / 720.0)
    for c in (1.0 / 120.0, 1.0 / 24.0, 1.0 / 6.0, 0.5, 1.0, 1.0):
        p = p * r + f(c)
    scale = ((np.clip(k, -126, 127).astype(np.int32) + 127) << 23).view(f)
    return np.where(x < f(-87.0), f(0.0), p * scale).astype(f)


def elementwise(x: torch.Tensor, op: int, alpha: float, beta: float) -> torch.Tensor:
    """Unary elementwise operators of the indexer on bf16 values (indexer/triton_kernels/elementwise_impl.py:
    62-104; op numbering of utils.py ElementwiseOpType: 0 relu form, 1 sigmoid, 2 silu, 3 abs, 4 add_mul).

    alpha and beta are rounded to bf16 first; every bf16 operation rounds once
    (z = bf16(bf16(beta * x) + alpha)); the logistic forms compute 1 / (1 + exp(z)) resp. x / (1 + exp(z)) in
    fp32 with `exp_canonical` (+inf above 88) and round once.  The reference leaves the rounding of
    beta * x + alpha and its exp to the Triton compiler: parity unpinned for ops 1, 2 and for op 3 / 4 with
    beta != 1; ops 0 and the default Abs are exact in any order.
    """
    assert x.dtype == torch.bfloat16
    f = np.float32
    a = f(torch.tensor(alpha).bfloat16().float().item())
    b = f(torch.tensor(beta).bfloat16().float().item())
    xv = x.float().numpy().astype(f)
    if op == 0:
        out = np.where(xv >= a, xv, b)
    else:
        z = torch.from_numpy(b * xv).bfloat16().float().numpy()
        z = torch.from_numpy(z + a).bfloat16().float().numpy()
        if op in (1, 2):
            with np.errstate(over="ignore", invalid="ignore"):
                e = np.where(z > f(88.0), f(np.inf), exp_canonical(np.minimum(z, f(88.0))))
                num = f(1.0) if op == 1 else xv
                out = (num / (f(1.0) + e)).astype(f)
        elif op == 3:
            out = np.abs(z)
        else:
            out = z
    return torch.from_numpy(np.asarray(out, dtype=f)).bfloat16()


def elementwise_binary(x: torch.Tensor, y: torch.Tensor, op: int, alpha: float = 1.0, beta: float = 1.0) -> torch.Tensor:
    """Binary elementwise operators on bf16 RAGGED tensors ``[rows, C, D]`` with broadcasting of the inner dims
    (indexer/triton_kernels/elementwise_binary_impl.py:72-86): 0 max, 1 min,
    2 bf16(bf16(alpha x) + bf16(beta y)), 3 bf16(x y); alpha and beta rounded to bf16 first."""
    assert x.dtype == y.dtype == torch.bfloat16
    xf, yf = torch.broadcast_tensors(x.float(), y.float())
    if op == 0:
        out = torch.maximum(xf, yf)
    elif op == 1:
        out = torch.minimum(xf, yf)
    elif op == 2:
        a = torch.tensor(alpha).bfloat16().float()
        b = torch.tensor(beta).bfloat16().float()
        out = (a * xf).bfloat16().float() + (b * yf).bfloat16().float()
    else:
        out = xf * yf
    return out.bfloat16()


def canonical_sum128(v: np.ndarray) -> np.float32:
    """Sum of a vector in the order the kernels use: 128 partial sums (element i goes to partial i % 128,
    added in ascending i from +0.0), then folded in halves v[j] += v[j + w], w = 64 .. 1."""
    f = np.float32
    n = len(v)
    pad = (-n) % 128
    a = np.concatenate([np.asarray(v, dtype=f), np.zeros(pad, dtype=f)]).reshape(-1, 128)
    part = np.zeros(128, dtype=f)
    for row in a:
        part = part + row
    w = 64
    while w >= 1:
        part = part[:w] + part[w:2 * w]
        w //= 2
    return part[0]


def candidate_windows(dense_indptr, eff_bs: int, topk_val: int, bos: int, eos: int):
    """Packed row ranges the indexer operators work on: the non-reserved candidates
    ``[indptr[s] + bos, indptr[s+1] - eos)`` of every segment that has more than ``topk_val`` of them
    (the planner's workload windows, csrc/utils_sglang.cu:219-251)."""
    for s in range(eff_bs):
        a = int(dense_indptr[s]) + bos
        b = int(dense_indptr[s + 1]) - eos
        if b - a > topk_val:
            yield s, a, b


def gemm_bpr(q, table, dense_indptr, dense_indices, eff_bs, topk_val, bos, eos,
             out: Optional[torch.Tensor] = None, rounding: str = "rne") -> torch.Tensor:
    """The ``GeMM`` indexer operator on (BATCHED, PAGED) inputs (indexer/matmul.py:194-399 over
    ``mm_bpr_kernel``, indexer/triton_kernels/matmul_impl.py:6-113): ``out[p, c, g] = table[row_p, c, :] . q[s, g, :]``
    for every candidate position p of segment s, bf16 values widened to fp32, fp32 products and sum (canonical
    order of `canonical_dot`), one rounding to bf16.  q [S, G, D], table [R, C, D] -> [N, C, G]."""
    assert q.dtype == torch.bfloat16 and table.dtype == torch.bfloat16
    total = int(dense_indptr[eff_bs])
    G, C = q.shape[1], table.shape[1]
    if out is None:
        out = torch.zeros(total, C, G, dtype=torch.bfloat16)
    for s, a, b in candidate_windows(dense_indptr, eff_bs, topk_val, bos, eos):
        rows = table[torch.as_tensor(np.asarray(dense_indices[a:b]), dtype=torch.long)].to(torch.float32)
        for c in range(C):
            for g in range(G):
                dot = canonical_dot(rows[:, c], q[s, g].to(torch.float32), bf16_products=False)
                out[a:b, c, g] = _round_bf16(dot, rounding)
    return out


def softmax_ragged(x, dense_indptr, eff_bs, topk_val, bos, eos, scale: float, rounding: str = "rne") -> torch.Tensor:
    """The in-place ``Softmax(dim=0, scale)`` indexer operator (indexer/scan.py over
    ``softmax_inplace_r_kernel``, indexer/triton_kernels/softmax_impl.py:6-105): for every inner element
    [r, c] of the RAGGED tensor x [N, r, c], softmax of ``scale * x`` over the candidate pages of each
    segment, rounded to bf16.  Canonical arithmetic: t = fp32(x) * scale, m = max t, e = `exp_canonical`(t - m),
    l = `canonical_sum128`(e), result = bf16(e / l).  (The reference accumulates (m, l) in blocks of 256
    pages with rescaling and uses the compiler's exp: same value up to rounding.)"""
    assert x.dtype == torch.bfloat16
    sc32 = np.float32(scale)
    N, R, C = x.shape
    for s, a, b in candidate_windows(dense_indptr, eff_bs, topk_val, bos, eos):
        blk = x[a:b].to(torch.float32).numpy()
        res = np.empty_like(blk)
        for r in range(R):
            for c in range(C):
                t = blk[:, r, c].astype(np.float32) * sc32
                e = exp_canonical(t - t.max())
                l = canonical_sum128(e)
                res[:, r, c] = (e / l).astype(np.float32)
        x[a:b] = _round_bf16(torch.from_numpy(res), rounding)
    return x


def canonical_sum_lastdim(vals: torch.Tensor) -> torch.Tensor:
    """fp32 sum over the last axis in the canonical order of `canonical_dot`: the axis is padded with +0.0 to
    a multiple of 8 and summed as chunks of 8 by L = min(32, pow2ceil(chunks)) partial sums folded in halves."""
    shape = vals.shape
    D = shape[-1]
    v = vals.reshape(-1, D).to(torch.float32)
    pad = (-D) % 8
    if pad:
        v = torch.cat([v, torch.zeros(v.shape[0], pad)], dim=1)
    return canonical_rowsum(v).reshape(shape[:-1])


REDUCE_MEAN, REDUCE_MAX, REDUCE_MIN, REDUCE_L2NORM, REDUCE_SUM = 0, 1, 2, 3, 4


def reduce_ragged(x, dim: int, kind: int, dense_indptr, eff_bs, topk_val, bos, eos,
                  out: Optional[torch.Tensor] = None, rounding: str = "rne") -> torch.Tensor:
    """The RAGGED reductions ``Mean / Max / Min / L2Norm / Sum (dim=1 | 2)`` of the indexer
    (indexer/reduce.py:165-309 over ``reduce_rr_kernel``, indexer/triton_kernels/reduce_impl.py:8-120):
    x [N, r, c] -> [N, 1, c] (dim 1) or [N, r, 1] (dim 2) on the candidate rows, fp32 arithmetic, one
    rounding to bf16.  Canonical orders: over dim 2 `canonical_sum_lastdim`; over dim 1 sequential in
    ascending order from +0.0.  Mean divides the sum by the axis length; L2Norm is the correctly rounded
    square root of the sum of the (exact) squares.  kind: REDUCE_* (the reference's ReduceType values)."""
    assert x.dtype == torch.bfloat16 and dim in (1, 2)
    N, R, C = x.shape
    if out is None:
        out = torch.zeros((N, 1, C) if dim == 1 else (N, R, 1), dtype=torch.bfloat16)
    for s, a, b in candidate_windows(dense_indptr, eff_bs, topk_val, bos, eos):
        blk = x[a:b].to(torch.float32)
        if kind == REDUCE_MAX:
            red = blk.max(dim=dim).values
        elif kind == REDUCE_MIN:
            red = blk.min(dim=dim).values
        else:
            v = blk * blk if kind == REDUCE_L2NORM else blk
            if dim == 2:
                red = canonical_sum_lastdim(v)
            else:
                red = torch.zeros(b - a, C, dtype=torch.float32)
                for r in range(R):
                    red = red + v[:, r]
            if kind == REDUCE_MEAN:
                red = red / float(blk.shape[dim])
            elif kind == REDUCE_L2NORM:
                red = torch.sqrt(red)
        out[a:b] = _round_bf16(red.unsqueeze(dim), rounding)
    return out


BINARY_MAX, BINARY_MIN, BINARY_ADD, BINARY_MUL = 0, 1, 2, 3


def binary_bpr(q, table, dense_indptr, dense_indices, eff_bs, topk_val, bos, eos, op: int, alpha: float = 1.0,
               beta: float = 1.0, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``Maximum / Minimum / Add / Multiply`` on (BATCHED, PAGED) inputs (indexer/elementwise_binary.py over
    ``elementwise_binary_bpr_kernel``, indexer/triton_kernels/elementwise_binary_impl.py:167-307):
    ``out[p] = op(q[s], table[row_p])`` with the inner dims broadcast, one rounding per bf16 operation
    (Add: bf16(bf16(alpha q) + bf16(beta y)) with alpha, beta rounded to bf16).  q [S, a0, a1],
    table [R, b0, b1] -> [N, max(a0, b0), max(a1, b1)]."""
    assert q.dtype == torch.bfloat16 and table.dtype == torch.bfloat16
    total = int(dense_indptr[eff_bs])
    d0, d1 = max(q.shape[1], table.shape[1]), max(q.shape[2], table.shape[2])
    if out is None:
        out = torch.zeros(total, d0, d1, dtype=torch.bfloat16)
    for s, a, b in candidate_windows(dense_indptr, eff_bs, topk_val, bos, eos):
        rows = table[torch.as_tensor(np.asarray(dense_indices[a:b]), dtype=torch.long)]
        out[a:b] = elementwise_binary(q[s:s + 1].expand(b - a, -1, -1), rows, op, alpha, beta)
    return out


def normalize_ragged(x, dense_indptr, eff_bs, topk_val, bos, eos, eps: float = 1e-12) -> torch.Tensor:
    """The in-place ``Normalize(dim=0)`` indexer operator (``normalize_inplace_r_kernel``,
    indexer/triton_kernels/normalize_impl.py:6-119): every inner element [r, c] divided by the L2 norm of
    that element over the candidate pages of its segment (at least eps), rounded to bf16.  Canonical
    arithmetic: exact squares, `canonical_sum128` over the pages, correctly rounded sqrt and division."""
    assert x.dtype == torch.bfloat16
    N, R, C = x.shape
    for s, a, b in candidate_windows(dense_indptr, eff_bs, topk_val, bos, eos):
        blk = x[a:b].to(torch.float32).numpy()
        res = np.empty_like(blk)
        for r in range(R):
            for c in range(C):
                v = blk[:, r, c].astype(np.float32)
                nrm = np.maximum(np.sqrt(canonical_sum128(v * v)), np.float32(eps)).astype(np.float32)
                res[:, r, c] = (v / nrm).astype(np.float32)
        x[a:b] = torch.from_numpy(res).to(torch.bfloat16)
    return x


def gqa_softmax_scores(q, centroids, dense_indptr, dense_indices, eff_bs, topk_val, bos, eos, scale: float,
                       out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Aggregated page scores of the ``gqa_block_sparse_attention`` flow (flow/algorithms.py:238-352):
    ``GeMM(q, centroids)`` -> ``Softmax(dim=0, scale)`` over the candidate pages -> ``Max(dim=2)`` over the
    query heads of the group, every operator output rounded to bf16 as in the reference: the composition
    of `gemm_bpr`, `softmax_ragged` and `reduce_ragged`."""
    assert q.dtype == torch.bfloat16, "this flow's operators are bf16 in the reference"
    args = (dense_indptr, eff_bs, topk_val, bos, eos)
    mm = gemm_bpr(q, centroids, dense_indptr, dense_indices, eff_bs, topk_val, bos, eos)
    softmax_ragged(mm, *args, scale)
    red = reduce_ragged(mm, 2, REDUCE_MAX, *args).view(-1)
    if out is None:
        return red
    out.view(-1)[: red.numel()] = red
    return out


def forward_indexer_gqa(q, centroids, plan, topk_val, bos, eos, scale: float = 0.09):
    """``GeMM -> Softmax -> Max -> topK`` of the gqa_block_sparse_attention flow; completes ``plan`` in place."""
    eff_bs = q.shape[0]
    scores = gqa_softmax_scores(q, centroids, plan["dense_kv_indptr"], plan["dense_kv_indices"], eff_bs, topk_val,
                                bos, eos, scale)
    topk_select(scores, plan["dense_kv_indptr"], plan["sparse_kv_indptr"], plan["dense_kv_indices"],
                plan["sparse_kv_indices"], eff_bs, topk_val, bos, eos)
    return scores


# --------------------------------------------------------------------------- #
# gqa_quest_sparse_attention flow: min/max envelopes and their indexer
# --------------------------------------------------------------------------- #
def cminmax(x: torch.Tensor, out: torch.Tensor, loc: torch.Tensor, page_size: int, num_kv_heads: int,
            op: str) -> None:
    """Page-completion ``Max(dim=1)`` / ``Min(dim=1)`` cache ops (cache/triton_kernels/reduce_impl.py:21-47,
    REDUCE_TYPE 1 / 2): same trigger and addressing as `cmean`; the reduction is exact in any order."""
    for t in loc.tolist():
        if (t + 1) % page_size != 0:
            continue
        for h in range(num_kv_heads):
            pid = (t // page_size) * num_kv_heads + h
            blk = x[pid].to(torch.float32)
            red = blk.max(dim=0).values if op == "max" else blk.min(dim=0).values
            out[pid, 0] = red.to(out.dtype)


def _cache_items(loc, page_size: int, num_kv_heads: int):
    """(paged row, ragged row) of every (slot of loc that closes a page, head): the blocks a cache-side
    operator touches (cache/triton_kernels/reduce_impl.py:21-32, 139-152, 260-275 of the reference)."""
    for i, t in enumerate(loc.tolist()):
        if (t + 1) % page_size != 0:
            continue
        for h in range(num_kv_heads):
            yield (t // page_size) * num_kv_heads + h, i * num_kv_heads + h


def cache_reduce(x, out, loc, page_size, num_kv_heads, dim: int, kind: int, x_ragged=False, out_ragged=False):
    """Cache-side ``Mean / Max / Min / L2Norm (dim)`` in every layout (cache/reduce.py:354-525 over
    reduce_pp / _rp / _pr / _rr): block [r, c] -> [1, c] (dim 1) or [r, 1] (dim 2).  fp32, canonical orders of
    `reduce_ragged` (rows: sequential; columns: `canonical_sum_lastdim`), one rounding."""
    for prow, rrow in _cache_items(loc, page_size, num_kv_heads):
        blk = x[rrow if x_ragged else prow].to(torch.float32)
        if kind == REDUCE_MAX:
            red = blk.max(dim=dim - 1).values
        elif kind == REDUCE_MIN:
            red = blk.min(dim=dim - 1).values
        else:
            v = blk * blk if kind == REDUCE_L2NORM else blk
            if dim == 2:
                red = canonical_sum_lastdim(v)
            else:
                red = torch.zeros(blk.shape[1], dtype=torch.float32)
                for r in range(blk.shape[0]):
                    red = red + v[r]
            red = red / float(blk.shape[dim - 1]) if kind == REDUCE_MEAN else torch.sqrt(red)
        out[rrow if out_ragged else prow] = red.to(out.dtype).view(out.shape[1:])
    return out


def cache_elementwise(x, out, loc, page_size, num_kv_heads, op, alpha, beta, x_ragged=False, out_ragged=False):
    """Cache-side ``Relu / Sigmoid / Silu / Abs / Add_Mul`` (cache/elementwise.py): `elementwise` on every
    triggered block."""
    for prow, rrow in _cache_items(loc, page_size, num_kv_heads):
        out[rrow if out_ragged else prow] = elementwise(x[rrow if x_ragged else prow], op, alpha, beta)
    return out


def cache_fill(x, loc, page_size, num_kv_heads, alpha):
    """Cache-side ``Fill`` (cache/fill.py:8-165 over fill_p_kernel, cache/triton_kernels/fill_impl.py:6-49): the
    whole block of every triggered (page, head) row of the PAGED tensor ``x`` becomes ``alpha`` rounded to x's
    dtype; nothing else changes.  In place."""
    for prow, _ in _cache_items(loc, page_size, num_kv_heads):
        x[prow] = torch.tensor(float(alpha), dtype=torch.float32).to(x.dtype)
    return x


def cache_binary(x, y, out, loc, page_size, num_kv_heads, op, alpha=1.0, beta=1.0, in_ragged=False, out_ragged=False):
    """Cache-side ``Maximum / Minimum / Add / Multiply`` (cache/elementwise_binary.py): `elementwise_binary` on
    every triggered pair of blocks."""
    for prow, rrow in _cache_items(loc, page_size, num_kv_heads):
        src = rrow if in_ragged else prow
        out[rrow if out_ragged else prow] = elementwise_binary(x[src:src + 1], y[src:src + 1], op, alpha, beta)[0]
    return out


def cache_gemm(x, y, out, loc, page_size, num_kv_heads, in_ragged=False, out_ragged=False):
    """Cache-side ``GeMM`` (cache/matmul.py over gemm_ppp / _ppr / _rrp / _rrr): ``O = Y X^T`` per triggered
    block, fp32 products, canonical sum over the inner dim, one rounding."""
    for prow, rrow in _cache_items(loc, page_size, num_kv_heads):
        src = rrow if in_ragged else prow
        xb, yb = x[src].to(torch.float32), y[src].to(torch.float32)
        prod = yb[:, None, :] * xb[None, :, :]                       # [ny, nx, k], exact for bf16 inputs
        out[rrow if out_ragged else prow] = canonical_sum_lastdim(prod).to(out.dtype)
    return out


def canonical_rowsum(vals: torch.Tensor) -> torch.Tensor:
    """Sum of every row of ``vals`` [R, D] (fp32) in the order of `canonical_dot` (chunks of 8, L partial
    sums taking chunks l, l+L, ..., folded in halves)."""
    R, D = vals.shape
    L = canonical_lanes(D)
    nch = D // 8
    v = vals.view(R, nch, 8)
    lane = torch.zeros(R, L, dtype=torch.float32)
    for c0 in range(0, nch, L):
        n = min(L, nch - c0)
        for j in range(8):
            lane[:, :n] = lane[:, :n] + v[:, c0:c0 + n, j]
    w = L // 2
    while w >= 1:
        lane = lane[:, :w] + lane[:, w:2 * w]
        w //= 2
    return lane[:, 0]


def quest_scores(q, cache_max, cache_min, dense_indptr, dense_indices, eff_bs, topk_val, bos, eos,
                 out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Aggregated page scores of the ``gqa_quest_sparse_attention`` flow (flow/algorithms.py:356-496):
    ``Multiply(q, max)`` and ``Multiply(q, min)`` (bf16 products), ``Maximum`` of the two, ``Sum(dim=2)`` over the
    head dim (fp32 sum, bf16 result), ``Max(dim=1)`` over the query heads: the composition of `binary_bpr`,
    `elementwise_binary` and `reduce_ragged`."""
    assert q.dtype == torch.bfloat16
    args = (dense_indptr, eff_bs, topk_val, bos, eos)
    hi = binary_bpr(q, cache_max, dense_indptr, dense_indices, eff_bs, topk_val, bos, eos, BINARY_MUL)
    lo = binary_bpr(q, cache_min, dense_indptr, dense_indices, eff_bs, topk_val, bos, eos, BINARY_MUL)
    u = elementwise_binary(hi, lo, BINARY_MAX)
    red = reduce_ragged(reduce_ragged(u, 2, REDUCE_SUM, *args), 1, REDUCE_MAX, *args).view(-1)
    if out is None:
        return red
    out.view(-1)[: red.numel()] = red
    return out


def forward_indexer_quest(q, cache_max, cache_min, plan, topk_val, bos, eos):
    """Indexer of the gqa_quest_sparse_attention flow; completes ``plan['sparse_kv_indices']`` in place."""
    eff_bs = q.shape[0]
    scores = quest_scores(q, cache_max, cache_min, plan["dense_kv_indptr"], plan["dense_kv_indices"], eff_bs,
                          topk_val, bos, eos)
    topk_select(scores, plan["dense_kv_indptr"], plan["sparse_kv_indptr"], plan["dense_kv_indices"],
                plan["sparse_kv_indices"], eff_bs, topk_val, bos, eos)
    return scores


# --------------------------------------------------------------------------- #
# prefill side: planners and chunk-wise transposes
# --------------------------------------------------------------------------- #
def plan_prefill(cached_seq_lens, input_seq_lens, req_to_token, req_indices, page_size: int, num_kv_heads: int):
    """Prefill planner (csrc/utils_sglang.cu:462-551): indptr of cached pages and of new query tokens in
    ragged (per request) and paged (per request and head) form, dense page list, last-page lengths and the
    token -> request table."""
    cached = np.asarray(cached_seq_lens, dtype=np.int64)
    inp = np.asarray(input_seq_lens, dtype=np.int64)
    r2t = np.asarray(req_to_token, dtype=np.int64)
    ridx = np.asarray(req_indices, dtype=np.int64)
    bs, H, P = len(cached), num_kv_heads, page_size
    n = (cached + P - 1) // P
    cn = np.concatenate([[0], np.cumsum(n)])
    ci = np.concatenate([[0], np.cumsum(inp)])
    kv_indptr = np.zeros(bs * H + 1, dtype=np.int32)
    qo_paged = np.zeros(bs * H + 1, dtype=np.int32)
    for r in range(bs):
        for j in range(H + 1):
            kv_indptr[r * H + j] = H * cn[r] + j * n[r]
            qo_paged[r * H + j] = H * ci[r] + j * inp[r]
    kv_indices = np.full(int(kv_indptr[-1]), NEG_FILL, dtype=np.int32)
    last = np.zeros(bs * H, dtype=np.int32)
    table = np.zeros(int(ci[-1]), dtype=np.uint16)
    for r in range(bs):
        toks = r2t[ridx[r]]
        ll = int(cached[r] % P)
        for h in range(H):
            s = r * H + h
            last[s] = P if ll == 0 else ll
            kv_indices[kv_indptr[s]:kv_indptr[s] + n[r]] = (toks[np.arange(n[r]) * P] // P) * H + h
        table[ci[r]:ci[r + 1]] = r
    return dict(dense_kv_indptr=kv_indptr, dense_kv_indices=kv_indices, qo_indptr_ragged=ci.astype(np.int32),
                qo_indptr_paged=qo_paged, kv_last_page_len=last, batch_table=table)


def plan_prefill_fa3(cached_seq_lens_per_seg, cu_seqlens_q, req_to_token, req_indices, page_size: int,
                     num_kv_heads: int, page_table_stride: int, num_tokens: int):
    """Block-table prefill planner (csrc/utils_sglang.cu:797-834): per-segment page table rows and the
    token -> request table located at ``cu_seqlens_q[r*H] / H``."""
    cached = np.asarray(cached_seq_lens_per_seg, dtype=np.int64)
    cu = np.asarray(cu_seqlens_q, dtype=np.int64)
    r2t = np.asarray(req_to_token, dtype=np.int64)
    ridx = np.asarray(req_indices, dtype=np.int64)
    H, P = num_kv_heads, page_size
    bs = len(ridx)
    pt = np.full((bs * H, page_table_stride), NEG_FILL, dtype=np.int32)
    table = np.zeros(num_tokens, dtype=np.uint16)
    for r in range(bs):
        toks = r2t[ridx[r]]
        for h in range(H):
            s = r * H + h
            npg = int((cached[s] + P - 1) // P)
            pt[s, :npg] = (toks[np.arange(npg) * P] // P) * H + h
        q_len = int(cu[r * H + 1] - cu[r * H])
        o = int(cu[r * H] // H)
        table[o:o + q_len] = r
    return dict(page_table=pt, batch_table=table)


def chunkwise_nh2hn(x: torch.Tensor, indptr, num_kv_heads: int) -> torch.Tensor:
    """[N, H*G, D] token-major -> [N*H, G, D] with every request's tokens regrouped head-major
    (csrc/utils_sglang.cu:623-663)."""
    N, HG, D = x.shape
    H = num_kv_heads
    G = HG // H
    out = torch.empty(N * H, G, D, dtype=x.dtype)
    xv = x.view(N, H, G, D)
    for b in range(len(indptr) - 1):
        o, e = int(indptr[b]), int(indptr[b + 1])
        out[o * H:e * H] = xv[o:e].permute(1, 0, 2, 3).reshape((e - o) * H, G, D)
    return out


def chunkwise_hn2nh(x: torch.Tensor, indptr, num_kv_heads: int) -> torch.Tensor:
    """Inverse of `chunkwise_nh2hn` for a tensor [N*H, G, ...] -> [N, H*G, ...] (csrc/utils_sglang.cu:698-751)."""
    H = num_kv_heads
    N = x.shape[0] // H
    G = x.shape[1]
    tail = tuple(x.shape[2:])
    out = torch.empty((N, H * G) + tail, dtype=x.dtype)
    for b in range(len(indptr) - 1):
        o, e = int(indptr[b]), int(indptr[b + 1])
        blk = x[o * H:e * H].reshape((H, e - o, G) + tail)
        out[o:e] = blk.transpose(0, 1).reshape((e - o, H * G) + tail)
    return out
