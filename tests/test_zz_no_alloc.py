"""The split-KV decode entry point that allocates nothing.

Some users of the library cannot allocate device memory at the point where they call attention (an engine
that gave the whole GPU to its own pool at start-up; a decode loop that must not trigger the device-wide
synchronisation of an allocation).  For them `vtx_decode_gqa_splitkv_noalloc` keeps the split states in a
fixed array inside the library instead of a caller workspace.  This test calls it through the C ABI, twice
in a row (the array is shared by all calls and keeps the previous call's contents), and checks both
results against the entry point that takes a caller workspace.  It is collected last so that a failure
here cannot hide the other tests in a run that stops at the first failure.
"""
import ctypes
import math

import pytest
import torch

from oracle import vortex_oracle as vo
from vortex_torch import _cabi

from _util import DevicePlan, close, to_dev

pytestmark = pytest.mark.gpu


def _call_noalloc(q, k, v, out, indptr, indices, last, eff_bs, P, scale, splits):
    fn = _cabi.lib.vtx_decode_gqa_splitkv_noalloc
    _cabi._limits(q, kv=k.shape[0])  # a no-op unless the checked library is loaded
    return fn(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), indptr.data_ptr(), indices.data_ptr(),
              last.data_ptr(), eff_bs, q.shape[1], q.shape[2], P, ctypes.c_float(scale), splits, _cabi.VTX_BF16,
              torch.cuda.current_stream().cuda_stream)


def test_noalloc_matches_workspace_variant_twice_in_a_row():
    H, G, D, P, K = 8, 2, 128, 16, 30
    scale = 1.0 / math.sqrt(D)
    outs = []
    for call, (seq, splits) in enumerate([([4096, 700, 33], 4), ([1500, 16, 2048, 5000], 3)]):
        prob = vo.make_paged_problem(60 + call, seq, H, G, D, P)
        dp = DevicePlan(prob, P, H, K, 1, 1)
        d = to_dev(prob)
        ws = torch.empty(_cabi.splitkv_workspace_bytes(dp.S, G, D, splits) // 4, device="cuda")
        want = torch.empty_like(d["q"])
        _cabi.decode_gqa_splitkv(d["q"], d["k"], d["v"], want, dp.dense_indptr, dp.dense_indices, dp.last_page_len,
                                 dp.S, P, scale, splits, ws)
        got = torch.full_like(d["q"], float("nan"))
        torch.cuda.synchronize()
        # Every buffer of this call exists now.  The entry point must not go through torch's allocator, which
        # would show in torch's reservation.  (The driver's free-memory count is no use as a check here: on a
        # shared GPU other processes move it too.  That the entry point calls no cudaMalloc is a property of
        # its source: it only launches kernels on a pointer obtained from cudaGetSymbolAddress.)
        reserved_before = torch.cuda.memory_reserved()
        rc = _call_noalloc(d["q"], d["k"], d["v"], got, dp.dense_indptr, dp.dense_indices, dp.last_page_len, dp.S,
                           P, scale, splits)
        torch.cuda.synchronize()
        assert rc == 0, _cabi.status_string(rc)
        assert torch.cuda.memory_reserved() == reserved_before
        assert close(got, want, 2e-2), f"call {call}: max err {(got.float() - want.float()).abs().max()}"
        oracle = vo.decode_gqa(prob["q"], prob["k"], prob["v"], dp.oracle(prob)["dense_kv_indptr"],
                               dp.oracle(prob)["dense_kv_indices"], dp.oracle(prob)["kv_last_page_len"])
        assert close(got, oracle, 2e-2)
        outs.append(got)
    assert not torch.isnan(outs[0].float()).any() and not torch.isnan(outs[1].float()).any()


def test_noalloc_refuses_requests_beyond_its_buffer():
    z = torch.zeros(8, dtype=torch.int32, device="cuda")
    q = torch.zeros(1, 2, 128, dtype=torch.bfloat16, device="cuda")
    kv = torch.zeros(1, 16, 128, dtype=torch.bfloat16, device="cuda")
    # 4096 segments x 64 splits x 2 heads x 130 floats is far more than the 8 MB array
    rc = _call_noalloc(q, kv, kv, q.clone(), z, z, z, 4096, 16, 0.1, 64)
    assert rc == 4 and "scratch" in _cabi.status_string(rc)
