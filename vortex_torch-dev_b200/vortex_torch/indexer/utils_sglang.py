"""Per-step planners called by the serving engine's attention backend.

Same call signatures as the reference's ``indexer/utils_sglang.py:15-44`` (``plan_decode``) and
``:135-171`` (``plan_decode_fa3``, the block-table form); both run as one kernel launch through
the C ABI.  The prefill-side helpers of the reference module are not part of the decode path
and raise ``NotImplementedError``.
"""
from __future__ import annotations

import torch

from .. import _cabi
from .context import Context


def plan_decode(cached_seq_lens: torch.Tensor, req_to_token: torch.Tensor, req_indices: torch.Tensor,
                ctx: Context) -> None:
    _cabi.plan_decode(
        cached_seq_lens, req_to_token, req_indices,
        ctx.dense_kv_indptr, ctx.dense_kv_indices, ctx.sparse_kv_indptr, ctx.sparse_kv_indices,
        ctx.kv_last_page_len, ctx.winfo_q_indices, ctx.winfo_kv_offsets, ctx.winfo_kv_lens,
        ctx.winfo_num_workloads, ctx.winfo_chunk_size, ctx.page_size, ctx.num_kv_heads, ctx.topk_val,
        ctx.page_reserved_bos, ctx.page_reserved_eos, ctx.max_chunk_size, ctx.min_chunk_size)
    ctx.set_batch_size(cached_seq_lens.shape[0])


def plan_decode_fa3(cached_seq_lens: torch.Tensor, req_to_token: torch.Tensor, req_indices: torch.Tensor,
                    dense_page_table: torch.Tensor, dense_cache_seqlens: torch.Tensor,
                    sparse_page_table: torch.Tensor, sparse_cache_seqlens: torch.Tensor, ctx: Context) -> None:
    _cabi.plan_decode(
        cached_seq_lens, req_to_token, req_indices,
        ctx.dense_kv_indptr, ctx.dense_kv_indices, ctx.sparse_kv_indptr, ctx.sparse_kv_indices,
        ctx.kv_last_page_len, ctx.winfo_q_indices, ctx.winfo_kv_offsets, ctx.winfo_kv_lens,
        ctx.winfo_num_workloads, ctx.winfo_chunk_size, ctx.page_size, ctx.num_kv_heads, ctx.topk_val,
        ctx.page_reserved_bos, ctx.page_reserved_eos, ctx.max_chunk_size, ctx.min_chunk_size,
        dense_page_table, dense_cache_seqlens, sparse_page_table, sparse_cache_seqlens)
    ctx.set_batch_size(cached_seq_lens.shape[0])


def _prefill_only(name: str):
    def _raise(*_a, **_k):
        raise NotImplementedError(
            f"vortex_torch.indexer.utils_sglang.{name}: prefill-side helper, not built in the sm_100a "
            f"decode-path library")

    _raise.__name__ = name
    return _raise


plan_prefill = _prefill_only("plan_prefill")
plan_prefill_fa3 = _prefill_only("plan_prefill_fa3")
chunkwise_nh2hn_transpose = _prefill_only("chunkwise_nh2hn_transpose")
chunkwise_hn2nh_transpose = _prefill_only("chunkwise_hn2nh_transpose")
chunkwise_hn2nh_transpose_fa3 = _prefill_only("chunkwise_hn2nh_transpose_fa3")


def indices_to_page_table(page_table: torch.Tensor, ctx: Context) -> None:
    """No-op in the reference as well (``indexer/utils_sglang.py:190-194``)."""
    return None
