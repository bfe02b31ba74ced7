"""Per-step planners called by the serving engine's attention backend.

Same call signatures as the reference's ``indexer/utils_sglang.py:15-44`` (``plan_decode``) and
``:135-171`` (``plan_decode_fa3``, the block-table form); both run as one kernel launch through
the C ABI.  The prefill-side helpers (``:47-187``: planners and chunk-wise transposes) keep their
signatures as well.
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


def plan_prefill(cached_seq_lens, dense_kv_indptr, dense_kv_indices, input_seq_lens, qo_indptr_ragged,
                 qo_indptr_paged, kv_last_page_len, req_to_token, req_indices, batch_table, page_size: int,
                 num_kv_heads: int) -> None:
    _cabi.plan_prefill(cached_seq_lens, dense_kv_indptr, dense_kv_indices, input_seq_lens, qo_indptr_ragged,
                       qo_indptr_paged, kv_last_page_len, req_to_token, req_indices, batch_table, page_size,
                       num_kv_heads)


def plan_prefill_fa3(cached_seq_lens, cu_seqlens_q, req_to_token, req_indices, page_table, batch_table,
                     page_size: int, num_kv_heads: int) -> None:
    _cabi.plan_prefill_fa3(cached_seq_lens, cu_seqlens_q, req_to_token, req_indices, page_table, batch_table,
                           page_size, num_kv_heads)


def chunkwise_nh2hn_transpose(x, indptr, batch_table, num_qo_heads: int, num_kv_heads: int, head_dim: int):
    return _cabi.chunkwise_nh2hn(x, indptr, batch_table, num_qo_heads, num_kv_heads, head_dim)


def chunkwise_hn2nh_transpose(x, y, indptr, batch_table, num_qo_heads: int, num_kv_heads: int, head_dim: int):
    return _cabi.chunkwise_hn2nh(x, y, indptr, batch_table, num_qo_heads, num_kv_heads, head_dim)


def chunkwise_hn2nh_transpose_fa3(x, indptr, batch_table, num_qo_heads: int, num_kv_heads: int, head_dim: int):
    return _cabi.chunkwise_hn2nh(x, None, indptr, batch_table, num_qo_heads, num_kv_heads, head_dim)[0]


def indices_to_page_table(page_table: torch.Tensor, ctx: Context) -> None:
    """No-op in the reference as well (``indexer/utils_sglang.py:190-194``)."""
    return None
