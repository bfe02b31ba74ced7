"""Drop-in for the reference's pybind11 extension module ``vortex_torch_C`` (``csrc/register.cc:5-14``).

Same function names and positional signatures (``csrc/register.h:15-133``; for ``topk_output`` the
order of the definition, ``csrc/topk.cu:117-128``, which is what the Python callers use), taking
torch tensors and forwarding to the C ABI of ``libvortex_b200.so``.  The five prefill-side
functions are not part of the decode path and raise ``NotImplementedError``.
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


def _prefill_only(name):
    def _raise(*_a, **_k):
        raise NotImplementedError(f"vortex_torch_C.{name}: prefill-side function, not built in the sm_100a "
                                  f"decode-path library")

    _raise.__name__ = name
    return _raise


sglang_plan_prefill = _prefill_only("sglang_plan_prefill")
sglang_plan_prefill_fa3 = _prefill_only("sglang_plan_prefill_fa3")
Chunkwise_NH2HN_Transpose = _prefill_only("Chunkwise_NH2HN_Transpose")
Chunkwise_HN2NH_Transpose = _prefill_only("Chunkwise_HN2NH_Transpose")
Chunkwise_HN2NH_Transpose_FA3 = _prefill_only("Chunkwise_HN2NH_Transpose_FA3")
