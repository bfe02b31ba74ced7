"""The benchmark configurations' full sizes on the GPU, checked through size-independent properties (and against the oracle
where the oracle's vectorised forms finish in seconds)."""
import math

import numpy as np
import pytest
import torch

from oracle import vortex_oracle as vo
from vortex_torch import _cabi

pytestmark = pytest.mark.gpu


def test_config4a_page_completion_512_requests():
    """512 requests each finish one 16-token page; centroid [8, 128] written at a random row: bit-exact."""
    P, H, D, pages = 16, 8, 128, 4096
    g = torch.Generator().manual_seed(41)
    k = torch.randn(pages * H, P, D, generator=g).bfloat16()
    pg = torch.randperm(pages, generator=g)[:512]
    loc = pg * P + (P - 1)
    out = torch.zeros(pages * H, 1, D, dtype=torch.bfloat16, device="cuda")
    _cabi.cmean(k.cuda(), out, loc.cuda(), H, P)
    rows = (pg.view(-1, 1) * H + torch.arange(H).view(1, -1)).reshape(-1)
    want = torch.zeros(pages * H, 1, D, dtype=torch.bfloat16)
    want[rows, 0] = vo.cmean_pages(k, rows)
    assert torch.equal(out.cpu().view(torch.int16), want.view(torch.int16))


def test_config4b_prefill_32768_tokens():
    """Prefill of one 32768-token request: 2048 page centroids x 8 heads from every token slot: bit-exact."""
    P, H, D, pages = 16, 8, 128, 2048
    g = torch.Generator().manual_seed(42)
    k = torch.randn(pages * H, P, D, generator=g).bfloat16()
    perm = torch.randperm(pages, generator=g)
    loc = (perm.view(-1, 1) * P + torch.arange(P).view(1, -1)).reshape(-1)  # all 32768 slots, page order shuffled
    out = torch.zeros(pages * H, 1, D, dtype=torch.bfloat16, device="cuda")
    _cabi.cmean(k.cuda(), out, loc.cuda(), H, P)
    rows = torch.arange(pages * H)
    assert torch.equal(out.cpu()[:, 0].view(torch.int16), vo.cmean_pages(k, rows).view(torch.int16))


@pytest.mark.parametrize("pages", [128, 2048])
def test_config4b_prefill_write_and_centroids_in_one_call(pages):
    """Prefill of a 2048- and of a 32768-token request through vtx_set_kv_cmean (one launch up to 16384 (token,
    head) items, copy and reduction as two launches inside the call above that): caches and all pages x 8
    centroids equal set_kv followed by the mean, bit for bit, and equal the oracle."""
    P, H, D, extra = 16, 8, 128, 64
    g = torch.Generator().manual_seed(44)
    perm = torch.randperm(pages + extra, generator=g)[:pages]       # physical pages of the request, in token order
    loc = (perm.view(-1, 1) * P + torch.arange(P).view(1, -1)).reshape(-1)
    nk = torch.randn(pages * P, H, D, generator=g).bfloat16().cuda()
    nv = torch.randn(pages * P, H, D, generator=g).bfloat16().cuda()
    res = []
    for fused in (True, False):
        k = torch.zeros((pages + extra) * H, P, D, dtype=torch.bfloat16, device="cuda")
        v = torch.zeros_like(k)
        c = torch.zeros((pages + extra) * H, 1, D, dtype=torch.bfloat16, device="cuda")
        if fused:
            _cabi.set_kv_cmean(k, v, nk, nv, c, loc.cuda(), P)
        else:
            _cabi.set_kv(k, v, nk, nv, loc.cuda(), P)
            _cabi.cmean(k, c, loc.cuda(), H, P)
        res.append((k, v, c))
    for a, b in zip(*res):
        assert torch.equal(a.view(torch.int16), b.view(torch.int16))
    rows = (perm.view(-1, 1) * H + torch.arange(H).view(1, -1)).reshape(-1)
    want = vo.cmean_pages(res[0][0].cpu(), rows)
    assert torch.equal(res[0][2].cpu()[rows, 0].view(torch.int16), want.view(torch.int16))


def test_prefill_chunk_that_continues_and_leaves_partial_pages():
    """A chunked prefill: the chunk starts in the middle of a page written earlier (its first rows come from
    the cache), spans whole pages and ends in a partial one; two requests in one call."""
    P, H, D, pages = 16, 4, 128, 40
    g = torch.Generator().manual_seed(45)
    k0 = torch.randn(pages * H, P, D, generator=g).bfloat16()
    v0 = torch.randn(pages * H, P, D, generator=g).bfloat16()
    perm = torch.randperm(pages, generator=g)
    # request A: pages perm[0:6], chunk covers slots 5 .. 5+70; request B: pages perm[10:13], slots 0 .. 40
    slot = lambda pgs, a, b: torch.as_tensor([int(pgs[i // P]) * P + i % P for i in range(a, b)], dtype=torch.int64)
    loc = torch.cat([slot(perm[0:6], 5, 75), slot(perm[10:13], 0, 40)])
    nnz = loc.numel()
    nk = torch.randn(nnz, H, D, generator=g).bfloat16().cuda()
    nv = torch.randn(nnz, H, D, generator=g).bfloat16().cuda()
    res = []
    for fused in (True, False):
        k, v = k0.cuda(), v0.cuda()
        c = torch.zeros(pages * H, 1, D, dtype=torch.bfloat16, device="cuda")
        if fused:
            _cabi.set_kv_cmean(k, v, nk, nv, c, loc.cuda(), P)
        else:
            _cabi.set_kv(k, v, nk, nv, loc.cuda(), P)
            _cabi.cmean(k, c, loc.cuda(), H, P)
        res.append((k, v, c))
    for a, b in zip(*res):
        assert torch.equal(a.view(torch.int16), b.view(torch.int16))
    assert int((res[0][2].float().abs().sum(dim=(1, 2)) > 0).sum()) == (4 + 2) * H   # pages closed: 4 of A, 2 of B


def test_config2_layer_properties_at_full_batch():
    """bs64 x 8192 tokens, one layer: the one-launch layer equals the separate kernels bit for bit, is
    idempotent, and its selection is a sorted prefix under the (score desc, position asc) order."""
    from _util import DevicePlan

    bs, H, G, D, P, K, bos, eos, ctx = 64, 8, 2, 128, 16, 30, 1, 1, 8192
    pages_per_req = ctx // P
    num_pages = bs * pages_per_req
    g = torch.Generator().manual_seed(43)
    perm = torch.randperm(num_pages, generator=g)
    slots = (perm.view(bs, pages_per_req, 1) * P + torch.arange(P).view(1, 1, P)).view(bs, -1).to(torch.int32)
    prob = dict(seq_lens=np.full(bs, ctx, dtype=np.int32), req_to_token=slots.numpy(),
                req_indices=np.arange(bs, dtype=np.int64))
    dp = DevicePlan(prob, P, H, K, bos, eos)
    torch.manual_seed(43)
    k = torch.empty(num_pages * H, P, D, dtype=torch.bfloat16, device="cuda").normal_()
    v = torch.empty(num_pages * H, P, D, dtype=torch.bfloat16, device="cuda").normal_()
    cent = torch.zeros(num_pages * H, 1, D, dtype=torch.bfloat16, device="cuda")
    _cabi.cmean(k, cent, torch.arange(num_pages, device="cuda", dtype=torch.int64) * P + (P - 1), H, P)
    q = torch.randn(bs * H, G, D, device="cuda").bfloat16()
    scale = 1.0 / math.sqrt(D)
    sel_a, out_a = dp.sparse_indices.clone(), torch.empty_like(q)
    _cabi.indexer_fused(q, cent, dp.dense_indptr, dp.sparse_indptr, dp.dense_indices, sel_a, dp.S, K, bos, eos, dp.max_pages)
    _cabi.decode_gqa(q, k, v, out_a, dp.sparse_indptr, sel_a, dp.last_page_len, dp.S, P, scale)
    for _ in range(2):  # twice: idempotent
        sel_b, out_b = dp.sparse_indices.clone(), torch.empty_like(q)
        _cabi.sparse_layer_fused(q, cent, k, v, out_b, dp.dense_indptr, dp.sparse_indptr, dp.dense_indices, sel_b,
                                 dp.last_page_len, dp.S, P, K, bos, eos, dp.max_pages, scale)
        assert torch.equal(sel_a, sel_b) and torch.equal(out_a.view(torch.int16), out_b.view(torch.int16))
    # sorted-prefix property from the stand-alone GeMV scores
    qm = q.float().mean(1, keepdim=True).bfloat16()
    scores = torch.zeros(num_pages * H, dtype=torch.bfloat16, device="cuda")
    _cabi.gemv(qm, cent, scores, dp.dense_indptr, dp.dense_indices, dp.S, K, bos, eos)
    sc = scores.float().view(dp.S, pages_per_req)[:, bos:pages_per_req - eos]          # [S, 510] by position
    rows = dp.dense_indices.view(dp.S, pages_per_req)[:, bos:pages_per_req - eos].long()
    chosen = sel_a.view(dp.S, K + bos + eos)[:, bos:bos + K].long()
    pos = torch.argsort(rows, dim=1)
    chosen_pos = torch.gather(pos, 1, torch.searchsorted(torch.gather(rows, 1, pos), chosen))
    chosen_sc = torch.gather(sc, 1, chosen_pos)
    # descending scores, ties by ascending position
    assert bool((chosen_sc[:, :-1] >= chosen_sc[:, 1:]).all())
    tie = chosen_sc[:, :-1] == chosen_sc[:, 1:]
    assert bool((chosen_pos[:, :-1][tie] < chosen_pos[:, 1:][tie]).all())
    # nothing left out beats the last selected one
    mask = torch.ones_like(sc, dtype=torch.bool)
    mask.scatter_(1, chosen_pos, False)
    rest_max = torch.where(mask, sc, torch.full_like(sc, -float("inf"))).max(dim=1).values
    assert bool((rest_max <= chosen_sc[:, -1]).all())
    assert torch.isfinite(out_a.float()).all()
    # requests 0, 31 and 63 against the CPU oracle: selection bit-exact, attention within 2e-2
    for r in (0, 31, 63):
        rows_r = ((slots[r, ::P].long() // P).view(-1, 1) * H + torch.arange(H).view(1, -1)).reshape(-1)
        plan = vo.plan_decode([ctx], np.arange(ctx, dtype=np.int32).reshape(1, -1), [0], P, H, K, bos, eos, 64, 16)
        kk, vv, cc = k[rows_r.cuda()].cpu(), v[rows_r.cuda()].cpu(), cent[rows_r.cuda()].cpu()
        qi = q[r * H:(r + 1) * H].cpu()
        vo.forward_indexer(qi, cc, plan, K, bos, eos)
        got = sel_a.view(dp.S, K + bos + eos)[r * H:(r + 1) * H].reshape(-1).cpu().numpy()
        np.testing.assert_array_equal(got, rows_r.numpy()[plan["sparse_kv_indices"]])
        want = vo.decode_gqa(qi, kk, vv, plan["sparse_kv_indptr"], plan["sparse_kv_indices"], plan["kv_last_page_len"])
        err = (out_a[r * H:(r + 1) * H].float().cpu() - want.float()).abs()
        assert bool((err <= 2e-2 * want.float().abs().clamp(min=1)).all())


def test_config5_mla_full_batch_two_forms_and_properties():
    """Config-5 size (bs128, 34 pages of 64 tokens per request out of a 16384-token context): the tcgen05
    and the mma.sync forms of the MLA decode are independent implementations and must agree; plus two
    properties of attention that need no oracle: permuting a request's page list leaves the output unchanged,
    and a request whose pages all hold one repeated latent row returns that row's first 512 dims."""
    bs, Hq, Dl, Dv, P, npg = 128, 16, 576, 512, 64, 34
    g = torch.Generator(device="cuda").manual_seed(55)
    pool = bs * 64
    cache = torch.randn(pool, P, Dl, generator=g, device="cuda", dtype=torch.float32).bfloat16()
    table = torch.stack([torch.randperm(pool, generator=g, device="cuda")[:npg] for _ in range(bs)]).int()
    lens = torch.full((bs,), npg * P, dtype=torch.int32, device="cuda")
    lens[1] = npg * P - 37  # one ragged request
    const_row = torch.randn(Dl, generator=g, device="cuda").bfloat16()
    cache[table[0].long()] = const_row  # request 0 attends to one repeated row
    q = torch.randn(bs, Hq, Dl, generator=g, device="cuda", dtype=torch.float32).bfloat16()
    scale = 1.0 / math.sqrt(192.0)
    outs = {}
    for path in (0, 1):
        out = torch.empty(bs, Hq, Dv, dtype=torch.bfloat16, device="cuda")
        old = _cabi.set_mla_path(path)
        try:
            _cabi.decode_mla(q, cache, out, table, lens, P, scale)
        finally:
            _cabi.set_mla_path(old)
        outs[path] = out.float()
    assert _cabi.mla_fault_bits() == 0
    a, b = outs[0], outs[1]
    assert bool(((a - b).abs() <= 2e-2 * b.abs().clamp(min=1)).all()), f"forms differ by {(a - b).abs().max()}"
    assert bool(((a[0] - const_row[:Dv].float()).abs() <= 2e-2).all())
    perm = torch.randperm(npg, generator=g, device="cuda")
    table2 = table.clone()
    table2[2:] = table[2:, perm]  # full requests only: the ragged one keeps its last page last
    out2 = torch.empty(bs, Hq, Dv, dtype=torch.bfloat16, device="cuda")
    _cabi.decode_mla(q, cache, out2, table2, lens, P, scale)
    assert bool(((out2.float() - a).abs() <= 2e-2 * a.abs().clamp(min=1)).all())
