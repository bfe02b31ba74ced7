"""KV-head split on the device: a rank that owns heads [lo, hi) runs the same kernels on a pool of hi - lo heads.

One GPU plays the head shards one after the other (they share nothing, so running them in turn is the same
computation as running them on several GPUs).  The union of the shards' results must equal the unsharded run
bit for bit: block tables and selections after translating local rows to rows of the unsharded pool, the caches
after the token write, and the attention outputs.
"""
import math

import numpy as np
import pytest
import torch

from oracle import vortex_oracle as vo
from vortex_torch import _cabi
from vortex_torch.runtime import Shard, head_range, local_row_to_global, slice_heads

from _util import DevicePlan, to_dev

pytestmark = pytest.mark.gpu


def _run(prob, H, G, D, P, K, loc, nk, nv, split_workspace):
    dp = DevicePlan(prob, P, H, K, 1, 1)
    d = to_dev(prob)
    k, v, c = d["k"].clone(), d["v"].clone(), d["centroids"].clone()
    sel = dp.sparse_indices.clone()
    out = torch.full_like(d["q"], float("nan"))
    ws = None
    if split_workspace:
        n = _cabi.sparse_layer_workspace_bytes(dp.S, dp.max_pages, K, 1, 1)
        ws = torch.zeros(max(1, n // 4), dtype=torch.int32, device="cuda")
    _cabi.sparse_layer_fused(d["q"], c, k, v, out, dp.dense_indptr, dp.sparse_indptr, dp.dense_indices, sel,
                             dp.last_page_len, dp.S, P, K, 1, 1, dp.max_pages, 1.0 / math.sqrt(D), nk.cuda(), nv.cuda(),
                             loc.cuda(), workspace=ws)
    torch.cuda.synchronize()
    return dp, k, v, c, sel, out


@pytest.mark.parametrize("head_shards,split_workspace", [(2, False), (4, True), (8, False)])
def test_head_shards_reproduce_the_unsharded_layer(head_shards, split_workspace):
    seq, H, G, D, P, K = [4096, 700, 33, 9008, 16 * 40], 8, 4, 128, 16, 30
    prob = vo.make_paged_problem(81, seq, H, G, D, P)
    bs = len(seq)
    loc = torch.as_tensor([int(prob["req_to_token"][r, seq[r] - 1]) for r in range(bs)], dtype=torch.int64)
    g = torch.Generator().manual_seed(9)
    nk = torch.randn(bs, H, D, generator=g).bfloat16()
    nv = torch.randn(bs, H, D, generator=g).bfloat16()
    dp, k, v, c, sel, out = _run(prob, H, G, D, P, K, loc, nk, nv, split_workspace)
    sip = dp.sparse_indptr.cpu().numpy()
    sel_h = sel.cpu().numpy()
    for i in range(head_shards):
        lo, hi = head_range(H, head_shards, i)
        sh = Shard(tuple(range(bs)), lo, hi)
        local = dict(prob)
        for name in ("k", "v", "centroids"):
            local[name] = slice_heads(prob[name], H, lo, hi)
        local["q"] = slice_heads(prob["q"], H, lo, hi)
        dpl, kl, vl, cl, sell, outl = _run(local, hi - lo, G, D, P, K, loc, nk[:, lo:hi].contiguous(),
                                          nv[:, lo:hi].contiguous(), split_workspace)
        assert torch.equal(kl.view(torch.int16), slice_heads(k, H, lo, hi).view(torch.int16))
        assert torch.equal(vl.view(torch.int16), slice_heads(v, H, lo, hi).view(torch.int16))
        assert torch.equal(cl.view(torch.int16), slice_heads(c, H, lo, hi).view(torch.int16))
        assert torch.equal(outl.view(torch.int16), slice_heads(out, H, lo, hi).view(torch.int16))
        sipl = dpl.sparse_indptr.cpu().numpy()
        sell_h = local_row_to_global(sell.cpu().numpy().astype(np.int64), H, sh)
        for r in range(bs):
            for hl in range(hi - lo):
                a, b = sipl[r * (hi - lo) + hl], sipl[r * (hi - lo) + hl + 1]
                ga, gb = sip[r * H + lo + hl], sip[r * H + lo + hl + 1]
                np.testing.assert_array_equal(sell_h[a:b], sel_h[ga:gb])
    assert _cabi.device_status() == 0
