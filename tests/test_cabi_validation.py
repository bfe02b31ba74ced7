"""Argument validation of the C ABI, without a GPU.

Every entry point checks its pointers, sizes, enums and shapes on the host before it touches the CUDA runtime and
answers VTX_ERR_INVALID_ARGUMENT (1) or VTX_ERR_UNSUPPORTED (2).  A call that got as far as a launch would answer
VTX_ERR_CUDA (3) on a machine without a GPU, so "1 or 2" shows that the refusal came first.  The pointers passed
here are never dereferenced: they only have to be non-null.
"""
import ctypes as C

import pytest

from vortex_torch import _cabi

NOT_KERNELS = ("vtx_set_mla_path", "vtx_mla_fault_read")
ENTRY_POINTS = [n for n in _cabi.SIGNATURES if n not in NOT_KERNELS]
DUMMY = 4096  # a non-null "pointer"


def _args(name, fill):
    out = []
    for t in _cabi.SIGNATURES[name]:
        out.append(C.c_void_p(DUMMY) if t is C.c_void_p else (C.c_float(1.0) if t is C.c_float else t(fill)))
    out[-1] = C.c_void_p(0)  # the stream
    return out


@pytest.mark.parametrize("name", ENTRY_POINTS)
def test_null_pointers_are_refused(name):
    rc = getattr(_cabi.lib, name)(*[t(0) for t in _cabi.SIGNATURES[name]])
    assert rc == 1, _cabi.status_string(rc)


@pytest.mark.parametrize("name", ENTRY_POINTS)
def test_negative_sizes_are_refused(name):
    rc = getattr(_cabi.lib, name)(*_args(name, -1))
    assert rc == 1, _cabi.status_string(rc)


# the three planners are pure index arithmetic: any positive page size and head count is a valid call
SHAPED = [n for n in ENTRY_POINTS if not n.startswith("vtx_plan_")]


@pytest.mark.parametrize("name", SHAPED)
def test_sizes_no_kernel_is_built_for_are_refused_before_any_launch(name):
    # every integer 3: head_dim 3, page_size 3, dtype 3, op 3 ... no entry point accepts all of these together
    rc = getattr(_cabi.lib, name)(*_args(name, 3))
    assert rc in (1, 2), f"{name}: {rc} ({_cabi.status_string(rc)})"


def _layer_params(**kw):
    base = dict(q=DUMMY, summary=DUMMY, summary2=0, k_cache=DUMMY, v_cache=DUMMY, out=DUMMY, new_k=0, new_v=0, loc=0,
                dense_kv_indptr=DUMMY, sparse_kv_indptr=DUMMY, dense_kv_indices=DUMMY, sparse_kv_indices=DUMMY,
                kv_last_page_len=DUMMY, workspace=0, workspace_bytes=0, eff_batch_size=8, group_size=4, head_dim=128,
                page_size=16, num_kv_heads=0, topk_val=30, page_reserved_bos=1, page_reserved_eos=1,
                max_num_pages_per_request=64, score_mode=_cabi.SCORE_MEAN_DOT, flags=0, dtype=_cabi.VTX_BF16,
                sm_scale=0.1, softmax_scale=0.0)
    base.update(kw)
    return _cabi.SparseLayerParams(**base)


@pytest.mark.parametrize("bad", [
    dict(q=0), dict(out=0), dict(k_cache=0), dict(kv_last_page_len=0),
    dict(head_dim=96), dict(group_size=3), dict(page_size=0), dict(eff_batch_size=-1), dict(topk_val=-2),
    dict(dtype=_cabi.VTX_F32), dict(dtype=9), dict(score_mode=1), dict(score_mode=7),
    dict(score_mode=_cabi.SCORE_QUEST),                       # quest needs the second summary cache
    dict(new_k=DUMMY),                                        # a token write needs new_v, loc and the head count
    dict(new_k=DUMMY, new_v=DUMMY, loc=DUMMY, num_kv_heads=0),
    dict(workspace=DUMMY, workspace_bytes=-1),
])
def test_sparse_layer_params_are_validated(bad):
    p = _layer_params(**bad)
    rc = _cabi.lib.vtx_sparse_layer(C.byref(p), None)
    assert rc in (1, 2), f"{bad}: {rc} ({_cabi.status_string(rc)})"


def test_sparse_layer_null_params():
    assert _cabi.lib.vtx_sparse_layer(None, None) == 1


def test_checked_entry_points_of_the_normal_library():
    if _cabi.CHECKED:
        pytest.skip("the checked library is loaded")
    assert _cabi.lib.vtx_checked_build() == 0
    assert _cabi.lib.vtx_checked_set_limits(1, 1, 1, 1, None) == 2  # unsupported: this build carries no checks


def test_workspace_size_queries_refuse_bad_sizes():
    assert _cabi.lib.vtx_sparse_layer_workspace_bytes(-1, 64, 30, 1, 1) <= 0
    assert _cabi.lib.vtx_decode_gqa_splitkv_workspace_bytes(8, 4, 128, 0) <= 0


def test_layer_workspace_size_follows_the_chunk_rule():
    """Chunks of 768 candidates for batches of at most 384 segments, 512 above; no workspace when one chunk holds
    the longest segment; tickets padded to 256 bytes, K eight-byte keys per (segment, chunk)."""
    ws = _cabi.lib.vtx_sparse_layer_workspace_bytes
    K = 64
    assert ws(256, 2048, K, 1, 1) == 1024 + 256 * 3 * K * 8        # 2046 candidates -> 3 chunks of 768
    assert ws(2048, 2048, K, 1, 1) == 8192 + 2048 * 4 * K * 8      # -> 4 chunks of 512
    assert ws(512, 512, 30, 1, 1) == 0 and ws(512, 515, 30, 1, 1) > 0   # 510 candidates fit one chunk, 513 do not
    assert ws(64, 770, 30, 1, 1) == 0 and ws(64, 771, 30, 1, 1) > 0     # small batch: 768 fit, 769 do not
