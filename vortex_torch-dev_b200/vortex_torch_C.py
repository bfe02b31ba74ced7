"""Drop-in for the reference's pybind11 extension module ``vortex_torch_C`` (``csrc/register.cc:5-14``).

Same function names and positional signatures (``csrc/register.h:15-133``; for ``topk_output`` the
order of the definition, ``csrc/topk.cu:117-128``, which is what the Python callers use), taking
torch tensors and forwarding to the C ABI of ``libvortex_b200.so``.  The three transposes allocate and
return their outputs, as the reference's do.
"""
from __future__ import annotations

from vortex_torch import _cabi


def sglang_plan_decode(cached_seq_lens, dense_kv_indptr, dense_kv_indices, sparse_kv_indptr, sparse_kv_indices,
                       kv_last_page_len, req_to_token, req_indices, winfo_q_indices, winfo_kv_offsets,
                       winfo_kv_lens, winfo_num_workloads, winfo_chunk_size, page_size, num_kv_heads, topk_val,
                       page_reserved_bos, page_reserved_eos, max_chunk_size, min_chunk_size):
    _cabi.plan_decode(cached_seq_lens, req_to_token, req_indices, dense_kv_indptr, dense_kv_indices,
                      sparse_kv_indptr, sparse_kv_indices, kv_last_page_len, winfo_q_indices, winfo_kv_offsets,
                      winfo_kv_lens, winfo_num_workloads, winfo_chunk_size, page_size, num_kv_heads, topk_val,
                      page_reserved_bos, page_reserved_eos, max_chunk_size, min_chunk_size)


def sglang_plan_decode_fa3(cached_seq_lens, dense_kv_indptr, dense_kv_indices, sparse_kv_indptr,
                           sparse_kv_indices, dense_page_table, dense_cache_seqlens, sparse_page_table,
                           sparse_cache_seqlens, req_to_token, req_indices, winfo_q_indices, winfo_kv_offsets,
                           winfo_kv_lens, winfo_num_workloads, winfo_chunk_size, page_size, num_kv_heads,
                           topk_val, page_reserved_bos, page_reserved_eos, max_chunk_size, min_chunk_size):
    _cabi.plan_decode(cached_seq_lens, req_to_token, req_indices, dense_kv_indptr, dense_kv_indices,
                      sparse_kv_indptr, sparse_kv_indices, None,  # this form has no kv_last_page_len output
                      winfo_q_indices, winfo_kv_offsets, winfo_kv_lens, winfo_num_workloads, winfo_chunk_size,
                      page_size, num_kv_heads, topk_val, page_reserved_bos, page_reserved_eos, max_chunk_size,
                      min_chunk_size, dense_page_table, dense_cache_seqlens, sparse_page_table,
                      sparse_cache_seqlens)


def topk_output(x, dense_kv_indptr, sparse_kv_indptr, dense_kv_indices, sparse_kv_indices, eff_batch_size,
                topk_val, reserved_bos, reserved_eos, max_num_pages):
    _cabi.topk(x, dense_kv_indptr, sparse_kv_indptr, dense_kv_indices, sparse_kv_indices, eff_batch_size,
               topk_val, reserved_bos, reserved_eos, max_num_pages)


def sglang_plan_prefill(cached_seq_lens, dense_kv_indptr, dense_kv_indices, input_seq_lens, qo_indptr_ragged,
                        qo_indptr_paged, kv_last_page_len, req_to_token, req_indices, batch_table, page_size,
                        num_kv_heads):
    _cabi.plan_prefill(cached_seq_lens, dense_kv_indptr, dense_kv_indices, input_seq_lens, qo_indptr_ragged,
                       qo_indptr_paged, kv_last_page_len, req_to_token, req_indices, batch_table, page_size,
                       num_kv_heads)


def sglang_plan_prefill_fa3(cached_seq_lens, cu_seqlens_q, req_to_token, req_indices, page_table, batch_table,
                            page_size, num_kv_heads):
    _cabi.plan_prefill_fa3(cached_seq_lens, cu_seqlens_q, req_to_token, req_indices, page_table, batch_table,
                           page_size, num_kv_heads)


def Chunkwise_NH2HN_Transpose(x, indptr, batch_table, num_qo_heads, num_kv_heads, head_dim):
    return _cabi.chunkwise_nh2hn(x, indptr, batch_table, num_qo_heads, num_kv_heads, head_dim)


def Chunkwise_HN2NH_Transpose(x, y, indptr, batch_table, num_qo_heads, num_kv_heads, head_dim):
    return _cabi.chunkwise_hn2nh(x, y, indptr, batch_table, num_qo_heads, num_kv_heads, head_dim)


def Chunkwise_HN2NH_Transpose_FA3(x, indptr, batch_table, num_qo_heads, num_kv_heads, head_dim):
    return _cabi.chunkwise_hn2nh(x, None, indptr, batch_table, num_qo_heads, num_kv_heads, head_dim)[0]
