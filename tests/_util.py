"""Shared helpers of the parity tests: move an oracle problem to the GPU and run the C-ABI path."""
from __future__ import annotations

import numpy as np
import torch

from oracle import vortex_oracle as vo
from vortex_torch import _cabi


class DevicePlan:
    """Device buffers of one planned decode step, filled through ``vtx_plan_decode``."""

    def __init__(self, prob, page_size, H, K, bos, eos, max_chunk=64, min_chunk=16, tables=False, device="cuda",
                 fill=-1):
        seq = torch.as_tensor(prob["seq_lens"], dtype=torch.int32, device=device)
        r2t = torch.as_tensor(prob["req_to_token"], dtype=torch.int32, device=device)
        ridx = torch.as_tensor(prob["req_indices"], dtype=torch.int64, device=device)
        bs = seq.shape[0]
        n = (np.asarray(prob["seq_lens"], dtype=np.int64) + page_size - 1) // page_size
        budget = K + bos + eos
        S = bs * H
        i32 = dict(dtype=torch.int32, device=device)
        self.bs, self.S, self.H, self.K, self.bos, self.eos, self.P = bs, S, H, K, bos, eos, page_size
        self.max_pages = int(n.max()) if bs else 1
        self.dense_indptr = torch.full((S + 1,), fill, **i32)
        self.sparse_indptr = torch.full((S + 1,), fill, **i32)
        self.dense_indices = torch.full((max(1, int(n.sum()) * H),), fill, **i32)
        self.sparse_indices = torch.full((max(1, int(np.minimum(n, budget).sum()) * H),), fill, **i32)
        self.last_page_len = torch.full((max(1, S),), fill, **i32)
        nw = max(1, int(n.sum()) * H // max(1, min_chunk) + S)
        self.w_q = torch.full((nw,), fill, **i32)
        self.w_off = torch.full((nw,), fill, **i32)
        self.w_len = torch.full((nw,), fill, **i32)
        self.w_num = torch.full((1,), fill, **i32)
        self.w_chunk = torch.full((1,), fill, **i32)
        self.tables = None
        if tables:
            stride = self.max_pages + 3
            self.tables = [torch.full((max(1, S), stride), fill, **i32), torch.full((max(1, S),), fill, **i32),
                           torch.full((max(1, S), stride), fill, **i32), torch.full((max(1, S),), fill, **i32)]
        t = self.tables or [None] * 4
        _cabi.plan_decode(seq, r2t, ridx, self.dense_indptr, self.dense_indices, self.sparse_indptr,
                          self.sparse_indices, self.last_page_len, self.w_q, self.w_off, self.w_len, self.w_num,
                          self.w_chunk, page_size, H, K, bos, eos, max_chunk, min_chunk, *t)
        self.max_chunk, self.min_chunk = max_chunk, min_chunk

    def oracle(self, prob):
        stride = None if self.tables is None else self.tables[0].shape[1]
        return vo.plan_decode(prob["seq_lens"], prob["req_to_token"], prob["req_indices"], self.P, self.H, self.K,
                              self.bos, self.eos, self.max_chunk, self.min_chunk, page_table_stride=stride)


def assert_plan_equal(dp: DevicePlan, ref: dict):
    S = dp.S
    np.testing.assert_array_equal(dp.dense_indptr.cpu().numpy()[:S + 1], ref["dense_kv_indptr"])
    np.testing.assert_array_equal(dp.sparse_indptr.cpu().numpy()[:S + 1], ref["sparse_kv_indptr"])
    nd, ns = int(ref["dense_kv_indptr"][-1]), int(ref["sparse_kv_indptr"][-1])
    np.testing.assert_array_equal(dp.dense_indices.cpu().numpy()[:nd], ref["dense_kv_indices"])
    np.testing.assert_array_equal(dp.sparse_indices.cpu().numpy()[:ns], ref["sparse_kv_indices"])
    np.testing.assert_array_equal(dp.last_page_len.cpu().numpy()[:S], ref["kv_last_page_len"])
    nw = int(ref["winfo_num_workloads"][0])
    assert int(dp.w_num.item()) == nw
    assert int(dp.w_chunk.item()) == int(ref["winfo_chunk_size"][0])
    np.testing.assert_array_equal(dp.w_q.cpu().numpy()[:nw], ref["winfo_q_indices"])
    np.testing.assert_array_equal(dp.w_off.cpu().numpy()[:nw], ref["winfo_kv_offsets"])
    np.testing.assert_array_equal(dp.w_len.cpu().numpy()[:nw], ref["winfo_kv_lens"])
    if dp.tables is not None:
        np.testing.assert_array_equal(dp.tables[0].cpu().numpy()[:S], ref["dense_page_table"])
        np.testing.assert_array_equal(dp.tables[1].cpu().numpy()[:S], ref["dense_cache_seqlens"])
        np.testing.assert_array_equal(dp.tables[2].cpu().numpy()[:S], ref["sparse_page_table"])
        np.testing.assert_array_equal(dp.tables[3].cpu().numpy()[:S], ref["sparse_cache_seqlens"])


def to_dev(prob, device="cuda"):
    return {k: (v.to(device) if isinstance(v, torch.Tensor) else v) for k, v in prob.items()}


def close(a: torch.Tensor, b: torch.Tensor, tol: float) -> bool:
    """|a-b| <= tol * max(1, |b|): the abs-or-rel acceptance rule of the attention outputs."""
    a, b = a.float().cpu(), b.float().cpu()
    return bool(((a - b).abs() <= tol * torch.clamp(b.abs(), min=1.0)).all())
