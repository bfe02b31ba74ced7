"""ctypes binding of ``libvortex_b200.so`` (the C ABI declared in ``include/vortex_b200.h``).

There is no fallback: if the library is missing the import fails, and every wrapper raises
``RuntimeError`` on a non-zero status.  Tensors are passed as raw device pointers and the
work is enqueued on torch's current CUDA stream.
"""
from __future__ import annotations

import ctypes as C
import os
from pathlib import Path

import torch

VTX_BF16, VTX_F32 = 0, 1

_PKG_ROOT = Path(__file__).resolve().parent.parent
# VORTEX_B200_CHECKED=1 loads the checked twin of the library (``build.py --checked``): same entry points, every
# index a kernel reads and then uses as an address compared with the sizes of the tensors the wrappers below see.
_CHECKED_ENV = os.environ.get("VORTEX_B200_CHECKED", "0") not in ("", "0")
LIB_PATH = Path(os.environ.get("VORTEX_B200_LIB", _PKG_ROOT / "lib" / (
    "libvortex_b200_checked.so" if _CHECKED_ENV else "libvortex_b200.so")))

if not LIB_PATH.exists():
    raise ImportError(
        f"vortex_torch: CUDA library {LIB_PATH} not found. Build it first with "
        f"`python {_PKG_ROOT / 'build.py'}` (needs nvcc with sm_100a support); there is no CPU fallback."
    )

lib = C.CDLL(str(LIB_PATH))

_p, _i, _i64, _f = C.c_void_p, C.c_int, C.c_int64, C.c_float

# name -> argument types, in header order
SIGNATURES = {
    "vtx_plan_decode": [_p, _p, _i64, _p] + [_p] * 10 + [_p] * 4 + [_i64] + [_i] * 8 + [_p],
    "vtx_set_kv": [_p, _p, _p, _p, _p, _i64, _i, _i, _i, _i, _p],
    "vtx_cmean": [_p, _p, _p, _i64, _i, _i, _i, _i, _i, _p],
    "vtx_creduce": [_p, _p, _p, _i64, _i, _i, _i, _i, _i, _i, _p],
    "vtx_indexer_quest_fused": [_p, _p, _p, _p, _p, _p, _p, _p, _i64, _i, _i, _i, _i, _i, _i, _i, _i, _p],
    "vtx_set_kv_cmean": [_p, _p, _p, _p, _p, _p, _i64, _i, _i, _i, _i, _p],
    "vtx_gemv": [_p, _p, _p, _p, _p, _i, _i, _i, _i, _i, _i, _p],
    "vtx_topk": [_p, _p, _p, _p, _p, _i, _i, _i, _i, _i, _i, _p],
    "vtx_indexer_fused": [_p, _p, _p, _p, _p, _p, _p, _i64, _i, _i, _i, _i, _i, _i, _i, _i, _p],
    "vtx_indexer_gqa_softmax_fused": [_p, _p, _p, _p, _p, _p, _p, _i64, _i, _i, _i, _i, _i, _i, _i, _f, _i, _p],
    "vtx_sparse_layer_fused": [_p] * 8 + [_i] + [_p] * 5 + [_i] * 8 + [_f, _i, _p],
    "vtx_sparse_layer_fused_gqa_softmax": [_p] * 8 + [_i] + [_p] * 5 + [_i] * 8 + [_f, _f, _i, _p],
    "vtx_sparse_layer_fused_quest": [_p] * 9 + [_i] + [_p] * 5 + [_i] * 8 + [_f, _i, _p],
    "vtx_decode_gqa": [_p, _p, _p, _p, _p, _p, _p, _i, _i, _i, _i, _f, _i, _p],
    "vtx_decode_gqa_splitkv": [_p, _p, _p, _p, _p, _p, _p, _i, _i, _i, _i, _f, _i, _p, _i64, _i, _p],
    "vtx_decode_gqa_splitkv_noalloc": [_p, _p, _p, _p, _p, _p, _p, _i, _i, _i, _i, _f, _i, _i, _p],
    "vtx_plan_prefill": [_p, _p, _p, _i64, _p, _p, _p, _p, _p, _p, _p, _i, _i, _i, _p],
    "vtx_plan_prefill_fa3": [_p, _p, _p, _i64, _p, _p, _i64, _p, _i, _i, _i, _p],
    "vtx_chunkwise_nh2hn": [_p, _p, _p, _p, _i64, _i, _i, _i, _p],
    "vtx_chunkwise_hn2nh": [_p, _p, _p, _p, _p, _p, _i64, _i, _i, _i, _p],
    "vtx_decode_mla": [_p, _p, _i64, _p, _p, _i64, _p, _i, _i, _i, _i, _i, _f, _i, _p],
    "vtx_mla_sparse_layer": [_p, _p, _p, _i64, _p, _p, _p, _p, _p, _p, _i64, _p] + [_i] * 9 + [_f, _i, _p],
    "vtx_elementwise": [_p, _p, _p, _i64, _i, _i, _f, _f, _i, _p],
    "vtx_elementwise_binary": [_p, _p, _p, _p, _i64, _i, _i, _i, _i, _i, _f, _f, _i, _p],
    "vtx_gemm_bpr": [_p, _p, _p, _p, _p, _i, _i, _i, _i, _i, _i, _i, _i, _p],
    "vtx_softmax_ragged": [_p, _p, _i, _i, _i, _i, _i, _f, _i, _p],
    "vtx_normalize_ragged": [_p, _p, _i, _i, _i, _i, _i, _f, _i, _p],
    "vtx_reduce_ragged": [_p, _p, _p, _i, _i, _i, _i, _i, _i, _i, _i, _i, _p],
    "vtx_binary_bpr": [_p, _p, _p, _p, _p, _i, _i, _i, _i, _i, _i, _f, _f, _i, _i, _i, _i, _i, _p],
    "vtx_transpose_ragged": [_p, _p, _p, _i, _i, _i, _i, _i, _i, _i, _p],
    "vtx_save_load_ragged": [_p, _p, _p, _p, _i, _i, _i, _i, _i, _i, _i, _p],
    "vtx_cache_reduce": [_p, _p, _p, _i64, _i, _i, _i, _i, _i, _i, _i, _i, _i, _p],
    "vtx_cache_elementwise": [_p, _p, _p, _i64, _i, _i, _i, _i, _f, _f, _i, _i, _i, _p],
    "vtx_cache_binary": [_p, _p, _p, _p, _i64, _i, _i, _i, _i, _i, _i, _i, _f, _f, _i, _i, _i, _p],
    "vtx_cache_gemm": [_p, _p, _p, _p, _i64, _i, _i, _i, _i, _i, _i, _i, _i, _p],
    "vtx_set_mla_path": [_i],
    "vtx_mla_fault_read": [_p],
}
for _name, _args in SIGNATURES.items():
    _fn = getattr(lib, _name)
    _fn.argtypes = _args
    _fn.restype = _i


class SparseLayerParams(C.Structure):
    """``vtx_sparse_layer_params`` of the header, field for field."""
    _fields_ = ([(n, _p) for n in ("q", "summary", "summary2", "k_cache", "v_cache", "out", "new_k", "new_v", "loc",
                                    "dense_kv_indptr", "sparse_kv_indptr", "dense_kv_indices", "sparse_kv_indices",
                                    "kv_last_page_len", "workspace")]
                + [("workspace_bytes", _i64)]
                + [(n, C.c_int32) for n in ("eff_batch_size", "group_size", "head_dim", "page_size", "num_kv_heads",
                                             "topk_val", "page_reserved_bos", "page_reserved_eos",
                                             "max_num_pages_per_request", "score_mode", "flags", "dtype")]
                + [("sm_scale", _f), ("softmax_scale", _f)])


SCORE_MEAN_DOT, SCORE_GQA_SOFTMAX, SCORE_QUEST = 0, 2, 3
LAYER_EARLY_PROLOGUE = 1
STATUS_CANDIDATE_OVERFLOW, STATUS_BAD_ROW = 1, 2

lib.vtx_sparse_layer.argtypes = [C.POINTER(SparseLayerParams), _p]
lib.vtx_sparse_layer.restype = _i
lib.vtx_sparse_layer_workspace_bytes.argtypes = [_i, _i, _i, _i, _i]
lib.vtx_sparse_layer_workspace_bytes.restype = _i64
lib.vtx_device_status_word.argtypes = []
lib.vtx_device_status_word.restype = _p
lib.vtx_device_status_read.argtypes = [_p, _i]
lib.vtx_device_status_read.restype = _i
lib.vtx_decode_gqa_splitkv_workspace_bytes.argtypes = [_i, _i, _i, _i]
lib.vtx_decode_gqa_splitkv_workspace_bytes.restype = _i64
lib.vtx_mla_fault_word.argtypes = []
lib.vtx_mla_fault_word.restype = _p
lib.vtx_checked_build.argtypes = []
lib.vtx_checked_build.restype = _i
lib.vtx_checked_set_limits.argtypes = [_i64, _i64, _i64, _i64, _p]
lib.vtx_checked_set_limits.restype = _i
lib.vtx_checked_get_limits.argtypes = [C.POINTER(_i64)]
lib.vtx_checked_get_limits.restype = _i
CHECKED = bool(lib.vtx_checked_build())
if _CHECKED_ENV and not CHECKED:
    raise ImportError(f"VORTEX_B200_CHECKED is set but {LIB_PATH} is not a checked build")
lib.vtx_set_programmatic_launch.argtypes = [_i]
lib.vtx_set_programmatic_launch.restype = _i
lib.vtx_version.restype = _i
lib.vtx_status_string.argtypes = [_i]
lib.vtx_status_string.restype = C.c_char_p
lib.vtx_last_cuda_error.restype = C.c_char_p

EXPORTED = sorted(list(SIGNATURES) + ["vtx_version", "vtx_status_string", "vtx_last_cuda_error",
                                    "vtx_set_programmatic_launch", "vtx_decode_gqa_splitkv_workspace_bytes",
                                    "vtx_mla_fault_word", "vtx_sparse_layer", "vtx_sparse_layer_workspace_bytes",
                                    "vtx_device_status_word", "vtx_device_status_read", "vtx_checked_build",
                                    "vtx_checked_set_limits", "vtx_checked_get_limits"])


def set_programmatic_launch(mode) -> None:
    """0/False off, anything else on (kernels are chained by programmatic dependent launch; each still waits
    for its whole predecessor).  Results are unchanged.  The early prologue of the fused layer kernel is a
    per-call flag of ``sparse_layer_fused`` (``early_prologue``)."""
    lib.vtx_set_programmatic_launch(int(mode))


def device_status(clear: bool = False) -> int:
    """The sticky status word of the kernels on the current device (``STATUS_*`` bits; 0 = nothing to report).
    Synchronises with the device."""
    host = C.c_uint32(0xFFFFFFFF)
    check(lib.vtx_device_status_read(C.byref(host), int(bool(clear))), "vtx_device_status_read")
    return int(host.value)


def sparse_layer_workspace_bytes(eff_bs: int, max_pages_per_request: int, topk_val: int, bos: int, eos: int) -> int:
    """Bytes of zero-initialised device scratch that lets ``sparse_layer_fused`` split long segments (0: no
    segment of that length is ever split)."""
    return int(lib.vtx_sparse_layer_workspace_bytes(int(eff_bs), int(max_pages_per_request), int(topk_val),
                                                    int(bos), int(eos)))


def version() -> int:
    return int(lib.vtx_version())


def status_string(code: int) -> str:
    return lib.vtx_status_string(int(code)).decode()


def check(code: int, what: str) -> None:
    if code != 0:
        extra = ""
        if code == 3:
            extra = ": " + lib.vtx_last_cuda_error().decode()
        raise RuntimeError(f"{what} failed with status {code} ({status_string(code)}{extra})")


def dtype_code(dt: torch.dtype) -> int:
    if dt == torch.bfloat16:
        return VTX_BF16
    if dt == torch.float32:
        return VTX_F32
    raise TypeError(f"vortex_b200 kernels take bfloat16 or float32 tensors, got {dt}")


def ptr(t) -> int:
    """Device pointer of a contiguous CUDA tensor (or 0 for None)."""
    if t is None:
        return 0
    if not t.is_cuda:
        raise RuntimeError("vortex_b200 kernels need CUDA tensors; there is no CPU fallback")
    if not t.is_contiguous():
        raise RuntimeError("vortex_b200 kernels need contiguous tensors")
    return t.data_ptr()


def stream_of(t: torch.Tensor) -> int:
    return torch.cuda.current_stream(t.device).cuda_stream


def _limits(ref: torch.Tensor, kv=None, summary=None, loc=None, req=None) -> None:
    """Checked build only: tell the kernels of the next launch on ``ref``'s stream how many rows the K/V cache
    (``kv``) and the page-summary cache (``summary``) have, how many token slots ``loc`` may address and how many
    rows the request-to-token table has.  None = unknown to this call = not compared."""
    if not CHECKED:
        return
    n = lambda v: -1 if v is None else int(v)
    check(lib.vtx_checked_set_limits(n(kv), n(summary), n(loc), n(req), stream_of(ref)), "vtx_checked_set_limits")


def checked_limits():
    """(kv_rows, summary_rows, loc_tokens, req_rows) in force on the device (checked library only)."""
    v = (_i64 * 4)()
    check(lib.vtx_checked_get_limits(v), "vtx_checked_get_limits")
    return tuple(int(x) for x in v)


def _slots(cache: torch.Tensor, num_kv_heads: int, page_size: int) -> int:
    """Token slots of a paged cache ``[pages * heads, ...]``."""
    return cache.shape[0] // max(1, int(num_kv_heads)) * int(page_size)


def _paged_slots(num_kv_heads: int, page_size: int, *operands):
    """Token slots that ``loc`` may address: the smallest PAGED operand decides (None if all are RAGGED)."""
    n = [_slots(t, num_kv_heads, page_size) for t, ragged in operands if t is not None and not ragged]
    return min(n) if n else None


def want(t: torch.Tensor, dt: torch.dtype, name: str) -> None:
    if t.dtype != dt:
        raise TypeError(f"{name} must be {dt}, got {t.dtype}")


# --------------------------------------------------------------------------- wrappers
def plan_decode(cached_seq_lens, req_to_token, req_indices, dense_kv_indptr, dense_kv_indices,
                sparse_kv_indptr, sparse_kv_indices, kv_last_page_len, winfo_q_indices, winfo_kv_offsets,
                winfo_kv_lens, winfo_num_workloads, winfo_chunk_size, page_size, num_kv_heads, topk_val,
                bos, eos, max_chunk_size, min_chunk_size, dense_page_table=None, dense_cache_seqlens=None,
                sparse_page_table=None, sparse_cache_seqlens=None) -> None:
    if cached_seq_lens.shape[0] == 0:  # an empty batch: nothing to do (torch hands out null pointers for empty tensors)
        return
    want(cached_seq_lens, torch.int32, "cached_seq_lens")
    want(req_to_token, torch.int32, "req_to_token")
    want(req_indices, torch.int64, "req_indices")
    for n, t in (("dense_kv_indptr", dense_kv_indptr), ("dense_kv_indices", dense_kv_indices),
                 ("sparse_kv_indptr", sparse_kv_indptr), ("sparse_kv_indices", sparse_kv_indices),
                 ("winfo_q_indices", winfo_q_indices),
                 ("winfo_kv_offsets", winfo_kv_offsets), ("winfo_kv_lens", winfo_kv_lens),
                 ("winfo_num_workloads", winfo_num_workloads), ("winfo_chunk_size", winfo_chunk_size)):
        want(t, torch.int32, n)
    if kv_last_page_len is not None:
        want(kv_last_page_len, torch.int32, "kv_last_page_len")
    stride = 0
    if dense_page_table is not None:
        for n, t in (("dense_page_table", dense_page_table), ("dense_cache_seqlens", dense_cache_seqlens),
                     ("sparse_page_table", sparse_page_table), ("sparse_cache_seqlens", sparse_cache_seqlens)):
            want(t, torch.int32, n)
        stride = dense_page_table.shape[1]
        if sparse_page_table.shape[1] != stride:
            raise ValueError("dense and sparse page tables must have the same row stride")
    _limits(cached_seq_lens, req=req_to_token.shape[0])
    rc = lib.vtx_plan_decode(
        ptr(cached_seq_lens), ptr(req_to_token), req_to_token.shape[1], ptr(req_indices),
        ptr(dense_kv_indptr), ptr(dense_kv_indices), ptr(sparse_kv_indptr), ptr(sparse_kv_indices),
        ptr(kv_last_page_len), ptr(winfo_q_indices), ptr(winfo_kv_offsets), ptr(winfo_kv_lens),
        ptr(winfo_num_workloads), ptr(winfo_chunk_size), ptr(dense_page_table), ptr(dense_cache_seqlens),
        ptr(sparse_page_table), ptr(sparse_cache_seqlens), stride, cached_seq_lens.shape[0],
        int(page_size), int(num_kv_heads), int(topk_val), int(bos), int(eos), int(max_chunk_size),
        int(min_chunk_size), stream_of(cached_seq_lens))
    check(rc, "vtx_plan_decode")


def set_kv(k_cache, v_cache, new_k, new_v, loc, page_size) -> None:
    if new_k.shape[0] == 0:  # an empty batch: nothing to do (torch hands out null pointers for empty tensors)
        return
    want(loc, torch.int64, "loc")
    nnz, H, D = new_k.shape
    _limits(k_cache, kv=k_cache.shape[0], loc=_slots(k_cache, H, page_size))
    rc = lib.vtx_set_kv(ptr(k_cache), ptr(v_cache), ptr(new_k), ptr(new_v), ptr(loc), nnz, H, D,
                        int(page_size), dtype_code(k_cache.dtype), stream_of(k_cache))
    check(rc, "vtx_set_kv")


def cmean(x, out, loc, num_kv_heads, page_size) -> None:
    if loc.shape[0] == 0:  # an empty batch: nothing to do (torch hands out null pointers for empty tensors)
        return
    want(loc, torch.int64, "loc")
    if out.dtype != x.dtype:
        raise TypeError("cmean: x and out must share a dtype")
    _limits(x, kv=x.shape[0], summary=out.shape[0], loc=_slots(x, num_kv_heads, page_size))
    rc = lib.vtx_cmean(ptr(x), ptr(out), ptr(loc), loc.shape[0], int(num_kv_heads), x.shape[1], x.shape[2],
                       int(page_size), dtype_code(x.dtype), stream_of(x))
    check(rc, "vtx_cmean")


def set_kv_cmean(k_cache, v_cache, new_k, new_v, centroids, loc, page_size) -> None:
    if new_k.shape[0] == 0:  # an empty batch: nothing to do (torch hands out null pointers for empty tensors)
        return
    want(loc, torch.int64, "loc")
    nnz, H, D = new_k.shape
    if not (k_cache.dtype == v_cache.dtype == new_k.dtype == new_v.dtype == centroids.dtype):
        raise TypeError("set_kv_cmean: caches, new tokens and centroids must share a dtype")
    _limits(k_cache, kv=k_cache.shape[0], summary=centroids.shape[0], loc=_slots(k_cache, H, page_size))
    rc = lib.vtx_set_kv_cmean(ptr(k_cache), ptr(v_cache), ptr(new_k), ptr(new_v), ptr(centroids), ptr(loc), nnz, H,
                              D, int(page_size), dtype_code(k_cache.dtype), stream_of(k_cache))
    check(rc, "vtx_set_kv_cmean")


def gemv(q_mean, centroids, scores, dense_kv_indptr, dense_kv_indices, eff_bs, topk_val, bos, eos) -> None:
    if int(eff_bs) == 0:  # an empty batch: nothing to do (torch hands out null pointers for empty tensors)
        return
    if not (q_mean.dtype == centroids.dtype == scores.dtype):
        raise TypeError("gemv: q_mean, centroids and scores must share a dtype")
    _limits(q_mean, summary=centroids.shape[0])
    rc = lib.vtx_gemv(ptr(q_mean), ptr(centroids), ptr(scores), ptr(dense_kv_indptr), ptr(dense_kv_indices),
                      int(eff_bs), q_mean.shape[-1], int(topk_val), int(bos), int(eos),
                      dtype_code(q_mean.dtype), stream_of(q_mean))
    check(rc, "vtx_gemv")


def topk(scores, dense_kv_indptr, sparse_kv_indptr, dense_kv_indices, sparse_kv_indices, eff_bs, topk_val,
         bos, eos, max_pages_per_request) -> None:
    if int(eff_bs) == 0:  # an empty batch: nothing to do (torch hands out null pointers for empty tensors)
        return
    want(sparse_kv_indices, torch.int32, "sparse_kv_indices")
    rc = lib.vtx_topk(ptr(scores), ptr(dense_kv_indptr), ptr(sparse_kv_indptr), ptr(dense_kv_indices),
                      ptr(sparse_kv_indices), int(eff_bs), int(topk_val), int(bos), int(eos),
                      int(max_pages_per_request), dtype_code(scores.dtype), stream_of(scores))
    check(rc, "vtx_topk")


def indexer_fused(q, centroids, dense_kv_indptr, sparse_kv_indptr, dense_kv_indices, sparse_kv_indices,
                  eff_bs, topk_val, bos, eos, max_pages_per_request, sparse_page_table=None) -> None:
    if int(eff_bs) == 0:  # an empty batch: nothing to do (torch hands out null pointers for empty tensors)
        return
    if q.dtype != centroids.dtype:
        raise TypeError("indexer_fused: q and centroids must share a dtype")
    stride = 0 if sparse_page_table is None else sparse_page_table.shape[1]
    _limits(q, summary=centroids.shape[0])
    rc = lib.vtx_indexer_fused(ptr(q), ptr(centroids), ptr(dense_kv_indptr), ptr(sparse_kv_indptr),
                               ptr(dense_kv_indices), ptr(sparse_kv_indices), ptr(sparse_page_table), stride,
                               int(eff_bs), q.shape[1], q.shape[2], int(topk_val), int(bos), int(eos),
                               int(max_pages_per_request), dtype_code(q.dtype), stream_of(q))
    check(rc, "vtx_indexer_fused")


def decode_gqa(q, k_cache, v_cache, out, kv_indptr, kv_indices, kv_last_page_len, eff_bs, page_size,
               sm_scale) -> None:
    if int(eff_bs) == 0:  # an empty batch: nothing to do (torch hands out null pointers for empty tensors)
        return
    if not (q.dtype == k_cache.dtype == v_cache.dtype == out.dtype):
        raise TypeError("decode_gqa: q, caches and out must share a dtype")
    _limits(q, kv=min(k_cache.shape[0], v_cache.shape[0]))
    rc = lib.vtx_decode_gqa(ptr(q), ptr(k_cache), ptr(v_cache), ptr(out), ptr(kv_indptr), ptr(kv_indices),
                            ptr(kv_last_page_len), int(eff_bs), q.shape[1], q.shape[2], int(page_size),
                            float(sm_scale), dtype_code(q.dtype), stream_of(q))
    check(rc, "vtx_decode_gqa")


def decode_mla(q, latent_cache, out, page_table, cache_seqlens, page_size, sm_scale) -> None:
    """q [bs, heads, latent_dim], latent_cache [rows, P, latent_dim], out [bs, heads, value_dim]."""
    if q.shape[0] == 0:  # an empty batch: nothing to do (torch hands out null pointers for empty tensors)
        return
    want(page_table, torch.int32, "page_table")
    want(cache_seqlens, torch.int32, "cache_seqlens")
    if not (q.dtype == latent_cache.dtype == out.dtype):
        raise TypeError("decode_mla: q, latent cache and out must share a dtype")
    rc = lib.vtx_decode_mla(ptr(q), ptr(latent_cache), latent_cache.shape[0], ptr(out), ptr(page_table),
                            page_table.shape[1], ptr(cache_seqlens), q.shape[0], q.shape[1], q.shape[2], out.shape[2], int(page_size),
                            float(sm_scale), dtype_code(q.dtype), stream_of(q))
    check(rc, "vtx_decode_mla")


def mla_sparse_layer(q, summary, latent_cache, out, dense_kv_indptr, sparse_kv_indptr, dense_kv_indices,
                     sparse_kv_indices, sparse_page_table, sparse_cache_seqlens, page_size, topk_val, bos, eos,
                     max_pages_per_request, sm_scale) -> None:
    """Page selection (as `indexer_fused` with ``sparse_page_table``) and `decode_mla` over the selected pages in
    one launch where the tcgen05 form allows it, else as the two launches; same results either way."""
    if q.shape[0] == 0:  # an empty batch: nothing to do (torch hands out null pointers for empty tensors)
        return
    want(sparse_page_table, torch.int32, "sparse_page_table")
    want(sparse_cache_seqlens, torch.int32, "sparse_cache_seqlens")
    if not (q.dtype == summary.dtype == latent_cache.dtype == out.dtype):
        raise TypeError("mla_sparse_layer: q, summary, latent cache and out must share a dtype")
    _limits(q, kv=latent_cache.shape[0], summary=summary.shape[0])
    rc = lib.vtx_mla_sparse_layer(ptr(q), ptr(summary), ptr(latent_cache), latent_cache.shape[0], ptr(out),
                                  ptr(dense_kv_indptr), ptr(sparse_kv_indptr), ptr(dense_kv_indices),
                                  ptr(sparse_kv_indices), ptr(sparse_page_table), sparse_page_table.shape[1],
                                  ptr(sparse_cache_seqlens), q.shape[0], q.shape[1], q.shape[2], out.shape[2],
                                  int(page_size), int(topk_val), int(bos), int(eos), int(max_pages_per_request),
                                  float(sm_scale), dtype_code(q.dtype), stream_of(q))
    check(rc, "vtx_mla_sparse_layer")


def elementwise(x, out, packed_row_count, op: int, alpha: float, beta: float) -> None:
    """Unary elementwise operator on the packed rows of a RAGGED tensor ``[S, C, D]`` (bf16);
    ``packed_row_count`` is a one-element int32 device tensor (a view of ``dense_kv_indptr[eff_bs:]``)."""
    want(packed_row_count, torch.int32, "packed_row_count")
    if x.dtype != out.dtype or x.shape != out.shape:
        raise TypeError("elementwise: x and out must share dtype and shape")
    rc = lib.vtx_elementwise(ptr(x), ptr(out), ptr(packed_row_count), x.shape[0], x.shape[1] * x.shape[2],
                             int(op), float(alpha), float(beta), dtype_code(x.dtype), stream_of(x))
    check(rc, "vtx_elementwise")


def elementwise_binary(x, y, out, packed_row_count, op: int, alpha: float = 1.0, beta: float = 1.0) -> None:
    """Binary elementwise operator on the packed rows of two RAGGED tensors (bf16), inner dims broadcast."""
    want(packed_row_count, torch.int32, "packed_row_count")
    if not (x.dtype == y.dtype == out.dtype):
        raise TypeError("elementwise_binary: x, y and out must share a dtype")
    if out.shape[1] != max(x.shape[1], y.shape[1]) or out.shape[2] != max(x.shape[2], y.shape[2]):
        raise ValueError("elementwise_binary: out must have the broadcast inner shape")
    rc = lib.vtx_elementwise_binary(ptr(x), ptr(y), ptr(out), ptr(packed_row_count), out.shape[0], x.shape[1],
                                    x.shape[2], y.shape[1], y.shape[2], int(op), float(alpha), float(beta),
                                    dtype_code(x.dtype), stream_of(x))
    check(rc, "vtx_elementwise_binary")


def set_mla_path(path: int) -> int:
    """0: tcgen05 form of the MLA decode where the page size allows (default); 1: mma.sync form."""
    return lib.vtx_set_mla_path(int(path))


def mla_fault_bits() -> int:
    """The sticky fault word of the tcgen05 MLA kernel (0 = no bounded wait ever gave up).  Synchronises."""
    host = C.c_uint32(0xFFFFFFFF)
    check(lib.vtx_mla_fault_read(C.byref(host)), "vtx_mla_fault_read")
    return int(host.value)


def sparse_layer_fused(q, centroids, k_cache, v_cache, out, dense_kv_indptr, sparse_kv_indptr, dense_kv_indices,
                       sparse_kv_indices, kv_last_page_len, eff_bs, page_size, topk_val, bos, eos,
                       max_pages_per_request, sm_scale, new_k=None, new_v=None, loc=None,
                       gqa_softmax_scale=None, quest_min=None, workspace=None, early_prologue=False) -> None:
    """Page selection and attention over the selected pages in one launch (bf16); with ``new_k``,
    ``new_v`` ``[bs, H, D]`` and ``loc`` ``[bs]`` the launch also writes the new token and the centroid
    of the page it closes.  ``gqa_softmax_scale`` set: page scores of the gqa_block_sparse_attention
    flow (per-head product, softmax over pages with that scale, maximum over heads) instead of the
    group-mean product.  ``quest_min`` set: page scores of the gqa_quest_sparse_attention flow with
    ``centroids`` as the per-page maximum cache and ``quest_min`` as the minimum cache (both are what a
    token write then maintains).  ``workspace``: zero-initialised device scratch of
    ``sparse_layer_workspace_bytes(...)`` bytes that lets long segments be scanned by several CTAs.
    ``early_prologue``: see ``VTX_LAYER_EARLY_PROLOGUE`` in the header."""
    if int(eff_bs) == 0:  # an empty batch: nothing to do (torch hands out null pointers for empty tensors)
        return
    if not (q.dtype == centroids.dtype == k_cache.dtype == v_cache.dtype == out.dtype):
        raise TypeError("sparse_layer_fused: q, centroids, caches and out must share a dtype")
    H = 0
    if new_k is not None:
        want(loc, torch.int64, "loc")
        H = new_k.shape[1]
        if new_k.dtype != q.dtype or new_v.dtype != q.dtype:
            raise TypeError("sparse_layer_fused: new_k/new_v must have q's dtype")
    mode = SCORE_QUEST if quest_min is not None else (SCORE_GQA_SOFTMAX if gqa_softmax_scale is not None
                                                     else SCORE_MEAN_DOT)
    p = SparseLayerParams(
        q=ptr(q), summary=ptr(centroids), summary2=ptr(quest_min), k_cache=ptr(k_cache), v_cache=ptr(v_cache),
        out=ptr(out), new_k=ptr(new_k), new_v=ptr(new_v), loc=ptr(loc), dense_kv_indptr=ptr(dense_kv_indptr),
        sparse_kv_indptr=ptr(sparse_kv_indptr), dense_kv_indices=ptr(dense_kv_indices),
        sparse_kv_indices=ptr(sparse_kv_indices), kv_last_page_len=ptr(kv_last_page_len),
        workspace=ptr(workspace),
        workspace_bytes=0 if workspace is None else workspace.numel() * workspace.element_size(),
        eff_batch_size=int(eff_bs), group_size=q.shape[1], head_dim=q.shape[2], page_size=int(page_size),
        num_kv_heads=H, topk_val=int(topk_val), page_reserved_bos=int(bos), page_reserved_eos=int(eos),
        max_num_pages_per_request=int(max_pages_per_request), score_mode=mode,
        flags=LAYER_EARLY_PROLOGUE if early_prologue else 0, dtype=dtype_code(q.dtype),
        sm_scale=float(sm_scale), softmax_scale=float(gqa_softmax_scale or 0.0))
    _limits(q, kv=min(k_cache.shape[0], v_cache.shape[0]),
            summary=centroids.shape[0] if quest_min is None else min(centroids.shape[0], quest_min.shape[0]),
            loc=None if new_k is None else _slots(k_cache, H, page_size))
    check(lib.vtx_sparse_layer(C.byref(p), stream_of(q)), "vtx_sparse_layer")


def splitkv_workspace_bytes(eff_bs: int, group: int, head_dim: int, num_splits: int) -> int:
    return int(lib.vtx_decode_gqa_splitkv_workspace_bytes(int(eff_bs), int(group), int(head_dim), int(num_splits)))


def decode_gqa_splitkv(q, k_cache, v_cache, out, kv_indptr, kv_indices, kv_last_page_len, eff_bs, page_size,
                       sm_scale, num_splits, workspace) -> None:
    """Split-KV form of `decode_gqa`; ``workspace`` is a device tensor of at least
    ``splitkv_workspace_bytes(...)`` bytes that the call overwrites."""
    if int(eff_bs) == 0:  # an empty batch: nothing to do (torch hands out null pointers for empty tensors)
        return
    if not (q.dtype == k_cache.dtype == v_cache.dtype == out.dtype):
        raise TypeError("decode_gqa_splitkv: q, caches and out must share a dtype")
    _limits(q, kv=min(k_cache.shape[0], v_cache.shape[0]))
    rc = lib.vtx_decode_gqa_splitkv(ptr(q), ptr(k_cache), ptr(v_cache), ptr(out), ptr(kv_indptr), ptr(kv_indices),
                                    ptr(kv_last_page_len), int(eff_bs), q.shape[1], q.shape[2], int(page_size),
                                    float(sm_scale), int(num_splits), ptr(workspace),
                                    workspace.numel() * workspace.element_size(), dtype_code(q.dtype), stream_of(q))
    check(rc, "vtx_decode_gqa_splitkv")


def indexer_gqa_softmax_fused(q, centroids, dense_kv_indptr, sparse_kv_indptr, dense_kv_indices, sparse_kv_indices,
                              eff_bs, topk_val, bos, eos, max_pages_per_request, softmax_scale,
                              sparse_page_table=None) -> None:
    """GeMM -> Softmax(scale) over pages -> Max over heads -> topK of the gqa_block_sparse_attention flow."""
    if int(eff_bs) == 0:  # an empty batch: nothing to do (torch hands out null pointers for empty tensors)
        return
    if q.dtype != centroids.dtype:
        raise TypeError("indexer_gqa_softmax_fused: q and centroids must share a dtype")
    stride = 0 if sparse_page_table is None else sparse_page_table.shape[1]
    _limits(q, summary=centroids.shape[0])
    rc = lib.vtx_indexer_gqa_softmax_fused(ptr(q), ptr(centroids), ptr(dense_kv_indptr), ptr(sparse_kv_indptr),
                                           ptr(dense_kv_indices), ptr(sparse_kv_indices), ptr(sparse_page_table),
                                           stride, int(eff_bs), q.shape[1], q.shape[2], int(topk_val), int(bos),
                                           int(eos), int(max_pages_per_request), float(softmax_scale),
                                           dtype_code(q.dtype), stream_of(q))
    check(rc, "vtx_indexer_gqa_softmax_fused")


def creduce(x, out, loc, num_kv_heads, page_size, op: int) -> None:
    """Page-completion reduction over rows: op 0 mean, 1 max, 2 min."""
    if loc.shape[0] == 0:  # an empty batch: nothing to do (torch hands out null pointers for empty tensors)
        return
    want(loc, torch.int64, "loc")
    if out.dtype != x.dtype:
        raise TypeError("creduce: x and out must share a dtype")
    _limits(x, kv=x.shape[0], summary=out.shape[0], loc=_slots(x, num_kv_heads, page_size))
    rc = lib.vtx_creduce(ptr(x), ptr(out), ptr(loc), loc.shape[0], int(num_kv_heads), x.shape[1], x.shape[2],
                         int(page_size), int(op), dtype_code(x.dtype), stream_of(x))
    check(rc, "vtx_creduce")


def indexer_quest_fused(q, cache_max, cache_min, dense_kv_indptr, sparse_kv_indptr, dense_kv_indices,
                        sparse_kv_indices, eff_bs, topk_val, bos, eos, max_pages_per_request,
                        sparse_page_table=None) -> None:
    """Multiply x2 -> Maximum -> Sum(dim=2) -> Max(dim=1) -> topK of the gqa_quest_sparse_attention flow."""
    if int(eff_bs) == 0:  # an empty batch: nothing to do (torch hands out null pointers for empty tensors)
        return
    if not (q.dtype == cache_max.dtype == cache_min.dtype):
        raise TypeError("indexer_quest_fused: q and the two caches must share a dtype")
    stride = 0 if sparse_page_table is None else sparse_page_table.shape[1]
    _limits(q, summary=min(cache_max.shape[0], cache_min.shape[0]))
    rc = lib.vtx_indexer_quest_fused(ptr(q), ptr(cache_max), ptr(cache_min), ptr(dense_kv_indptr),
                                     ptr(sparse_kv_indptr), ptr(dense_kv_indices), ptr(sparse_kv_indices),
                                     ptr(sparse_page_table), stride, int(eff_bs), q.shape[1], q.shape[2],
                                     int(topk_val), int(bos), int(eos), int(max_pages_per_request),
                                     dtype_code(q.dtype), stream_of(q))
    check(rc, "vtx_indexer_quest_fused")


def plan_prefill(cached_seq_lens, dense_kv_indptr, dense_kv_indices, input_seq_lens, qo_indptr_ragged,
                 qo_indptr_paged, kv_last_page_len, req_to_token, req_indices, batch_table, page_size,
                 num_kv_heads) -> None:
    for n, t in (("cached_seq_lens", cached_seq_lens), ("dense_kv_indptr", dense_kv_indptr),
                 ("dense_kv_indices", dense_kv_indices), ("input_seq_lens", input_seq_lens),
                 ("qo_indptr_ragged", qo_indptr_ragged), ("qo_indptr_paged", qo_indptr_paged),
                 ("kv_last_page_len", kv_last_page_len), ("req_to_token", req_to_token)):
        want(t, torch.int32, n)
    want(req_indices, torch.int64, "req_indices")
    want(batch_table, torch.uint16, "batch_table")
    _limits(cached_seq_lens, req=req_to_token.shape[0])
    rc = lib.vtx_plan_prefill(ptr(cached_seq_lens), ptr(input_seq_lens), ptr(req_to_token), req_to_token.shape[1],
                              ptr(req_indices), ptr(dense_kv_indptr), ptr(dense_kv_indices), ptr(qo_indptr_ragged),
                              ptr(qo_indptr_paged), ptr(kv_last_page_len), ptr(batch_table),
                              cached_seq_lens.shape[0], int(page_size), int(num_kv_heads), stream_of(cached_seq_lens))
    check(rc, "vtx_plan_prefill")


def plan_prefill_fa3(cached_seq_lens, cu_seqlens_q, req_to_token, req_indices, page_table, batch_table, page_size,
                     num_kv_heads) -> None:
    for n, t in (("cached_seq_lens", cached_seq_lens), ("cu_seqlens_q", cu_seqlens_q), ("req_to_token", req_to_token),
                 ("page_table", page_table)):
        want(t, torch.int32, n)
    want(req_indices, torch.int64, "req_indices")
    want(batch_table, torch.uint16, "batch_table")
    _limits(req_indices, req=req_to_token.shape[0])
    rc = lib.vtx_plan_prefill_fa3(ptr(cached_seq_lens), ptr(cu_seqlens_q), ptr(req_to_token), req_to_token.shape[1],
                                  ptr(req_indices), ptr(page_table), page_table.shape[1], ptr(batch_table),
                                  req_indices.shape[0], int(page_size), int(num_kv_heads), stream_of(req_indices))
    check(rc, "vtx_plan_prefill_fa3")


def chunkwise_nh2hn(x, indptr, batch_table, num_qo_heads, num_kv_heads, head_dim):
    want(x, torch.bfloat16, "x")
    want(indptr, torch.int32, "indptr")
    want(batch_table, torch.uint16, "batch_table")
    n, G = x.shape[0], num_qo_heads // num_kv_heads
    out = torch.empty((n * num_kv_heads, G, head_dim), dtype=x.dtype, device=x.device)
    rc = lib.vtx_chunkwise_nh2hn(ptr(x), ptr(out), ptr(indptr), ptr(batch_table), n, int(num_kv_heads), G,
                                 int(head_dim), stream_of(x))
    check(rc, "vtx_chunkwise_nh2hn")
    return out


def chunkwise_hn2nh(x, y, indptr, batch_table, num_qo_heads, num_kv_heads, head_dim):
    want(x, torch.bfloat16, "x")
    want(indptr, torch.int32, "indptr")
    want(batch_table, torch.uint16, "batch_table")
    n, G = x.shape[0] // num_kv_heads, x.shape[1]
    x_out = torch.empty((n, num_qo_heads, head_dim), dtype=x.dtype, device=x.device)
    y_out = None
    if y is not None:
        want(y, torch.float32, "y")
        y_out = torch.empty((n, num_qo_heads), dtype=y.dtype, device=y.device)
    rc = lib.vtx_chunkwise_hn2nh(ptr(x), ptr(x_out), ptr(y), ptr(y_out), ptr(indptr), ptr(batch_table), n,
                                 int(num_kv_heads), G, int(head_dim), stream_of(x))
    check(rc, "vtx_chunkwise_hn2nh")
    return x_out, y_out


# --------------------------------------------------------------------------- stand-alone chained operators
def _win(ctx):
    """(dense_kv_indptr, eff_bs, topk_val, bos, eos) of an indexer context."""
    return ctx.dense_kv_indptr, ctx.batch_size * ctx.num_kv_heads, ctx.topk_val, ctx.page_reserved_bos, \
        ctx.page_reserved_eos


def gemm_bpr(q, table, out, dense_kv_indptr, dense_kv_indices, eff_bs, topk_val, bos, eos) -> None:
    """``out[p, c, g] = table[row_p, c, :] . q[s, g, :]`` on every candidate row (bf16, fp32 products and sum)."""
    if not (q.dtype == table.dtype == out.dtype):
        raise TypeError("gemm_bpr: q, table and out must share a dtype")
    _limits(q, summary=table.shape[0])
    rc = lib.vtx_gemm_bpr(ptr(q), ptr(table), ptr(out), ptr(dense_kv_indptr), ptr(dense_kv_indices), int(eff_bs),
                          q.shape[1], table.shape[1], q.shape[2], int(topk_val), int(bos), int(eos),
                          dtype_code(q.dtype), stream_of(q))
    check(rc, "vtx_gemm_bpr")


def softmax_ragged(x, dense_kv_indptr, eff_bs, topk_val, bos, eos, scale: float) -> None:
    rc = lib.vtx_softmax_ragged(ptr(x), ptr(dense_kv_indptr), int(eff_bs), x.shape[1] * x.shape[2], int(topk_val),
                                int(bos), int(eos), float(scale), dtype_code(x.dtype), stream_of(x))
    check(rc, "vtx_softmax_ragged")


def normalize_ragged(x, dense_kv_indptr, eff_bs, topk_val, bos, eos, eps: float = 1e-12) -> None:
    rc = lib.vtx_normalize_ragged(ptr(x), ptr(dense_kv_indptr), int(eff_bs), x.shape[1] * x.shape[2], int(topk_val),
                                  int(bos), int(eos), float(eps), dtype_code(x.dtype), stream_of(x))
    check(rc, "vtx_normalize_ragged")


def reduce_ragged(x, out, dim: int, kind: int, dense_kv_indptr, eff_bs, topk_val, bos, eos) -> None:
    """kind: 0 mean, 1 max, 2 min, 3 l2norm, 4 sum over axis ``dim`` (1 or 2) of ``x`` ``[N, r, c]``."""
    rc = lib.vtx_reduce_ragged(ptr(x), ptr(out), ptr(dense_kv_indptr), int(eff_bs), x.shape[1], x.shape[2], int(dim),
                               int(kind), int(topk_val), int(bos), int(eos), dtype_code(x.dtype), stream_of(x))
    check(rc, "vtx_reduce_ragged")


def binary_bpr(q, table, out, dense_kv_indptr, dense_kv_indices, eff_bs, topk_val, bos, eos, op: int,
               alpha: float = 1.0, beta: float = 1.0, x_is_ragged: bool = False) -> None:
    """op 0 max, 1 min, 2 alpha q + beta y, 3 q y between ``q[s]`` (or, with ``x_is_ragged``, the RAGGED row
    ``q[p]``) and ``table[row_p]`` (inner dims broadcast)."""
    _limits(q, summary=table.shape[0])
    rc = lib.vtx_binary_bpr(ptr(q), ptr(table), ptr(out), ptr(dense_kv_indptr), ptr(dense_kv_indices), int(eff_bs),
                            q.shape[1], q.shape[2], table.shape[1], table.shape[2], int(op), float(alpha), float(beta),
                            int(bool(x_is_ragged)), int(topk_val), int(bos), int(eos), dtype_code(q.dtype), stream_of(q))
    check(rc, "vtx_binary_bpr")


def transpose_ragged(x, out, dense_kv_indptr, eff_bs, topk_val, bos, eos) -> None:
    rc = lib.vtx_transpose_ragged(ptr(x), ptr(out), ptr(dense_kv_indptr), int(eff_bs), x.shape[1], x.shape[2],
                                  int(topk_val), int(bos), int(eos), dtype_code(x.dtype), stream_of(x))
    check(rc, "vtx_transpose_ragged")


def save_load_ragged(ragged, paged, dense_kv_indptr, dense_kv_indices, eff_bs, topk_val, bos, eos, save: bool) -> None:
    _limits(ragged, summary=paged.shape[0])
    rc = lib.vtx_save_load_ragged(ptr(ragged), ptr(paged), ptr(dense_kv_indptr), ptr(dense_kv_indices), int(eff_bs),
                                  ragged.shape[1] * ragged.shape[2], int(bool(save)), int(topk_val), int(bos), int(eos),
                                  dtype_code(ragged.dtype), stream_of(ragged))
    check(rc, "vtx_save_load_ragged")


# --------------------------------------------------------------------------- cache-side operators, every layout
def cache_reduce(x, out, loc, num_kv_heads, page_size, dim: int, kind: int, x_ragged=False, out_ragged=False) -> None:
    """kind 0 mean, 1 max, 2 min, 3 l2norm over axis ``dim`` of the triggered blocks of ``x`` ``[*, r, c]``."""
    want(loc, torch.int64, "loc")
    _limits(x, loc=_paged_slots(num_kv_heads, page_size, (x, x_ragged), (out, out_ragged)))
    rc = lib.vtx_cache_reduce(ptr(x), ptr(out), ptr(loc), loc.shape[0], int(num_kv_heads), x.shape[1], x.shape[2],
                              int(page_size), int(dim), int(kind), int(bool(x_ragged)), int(bool(out_ragged)),
                              dtype_code(x.dtype), stream_of(x))
    check(rc, "vtx_cache_reduce")


def cache_elementwise(x, out, loc, num_kv_heads, page_size, op: int, alpha: float, beta: float, x_ragged=False,
                      out_ragged=False) -> None:
    want(loc, torch.int64, "loc")
    _limits(x, loc=_paged_slots(num_kv_heads, page_size, (x, x_ragged), (out, out_ragged)))
    rc = lib.vtx_cache_elementwise(ptr(x), ptr(out), ptr(loc), loc.shape[0], int(num_kv_heads),
                                   x.shape[1] * x.shape[2], int(page_size), int(op), float(alpha), float(beta),
                                   int(bool(x_ragged)), int(bool(out_ragged)), dtype_code(x.dtype), stream_of(x))
    check(rc, "vtx_cache_elementwise")


def cache_binary(x, y, out, loc, num_kv_heads, page_size, op: int, alpha: float = 1.0, beta: float = 1.0,
                 in_ragged=False, out_ragged=False) -> None:
    want(loc, torch.int64, "loc")
    _limits(x, loc=_paged_slots(num_kv_heads, page_size, (x, in_ragged), (y, in_ragged), (out, out_ragged)))
    rc = lib.vtx_cache_binary(ptr(x), ptr(y), ptr(out), ptr(loc), loc.shape[0], int(num_kv_heads), x.shape[1],
                              x.shape[2], y.shape[1], y.shape[2], int(page_size), int(op), float(alpha), float(beta),
                              int(bool(in_ragged)), int(bool(out_ragged)), dtype_code(x.dtype), stream_of(x))
    check(rc, "vtx_cache_binary")


def cache_gemm(x, y, out, loc, num_kv_heads, page_size, in_ragged=False, out_ragged=False) -> None:
    """``out block = y block . (x block)^T`` for every triggered (token, head)."""
    want(loc, torch.int64, "loc")
    _limits(x, loc=_paged_slots(num_kv_heads, page_size, (x, in_ragged), (y, in_ragged), (out, out_ragged)))
    rc = lib.vtx_cache_gemm(ptr(x), ptr(y), ptr(out), ptr(loc), loc.shape[0], int(num_kv_heads), x.shape[1],
                            y.shape[1], x.shape[2], int(page_size), int(bool(in_ragged)), int(bool(out_ragged)),
                            dtype_code(x.dtype), stream_of(x))
    check(rc, "vtx_cache_gemm")
