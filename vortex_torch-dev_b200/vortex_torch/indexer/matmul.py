"""``GeMV``: centroid scores for every candidate page (reference op: ``indexer/matmul.py:10-189``).

``GeMV()(x, y, ctx=ctx)`` with ``x`` BATCHED ``[S, 1, D]`` and ``y`` PAGED ``[num_pages*H, 1, D]``
returns a RAGGED ``[ctx.max_num_pages, 1, 1]`` buffer holding, at each candidate's packed dense
position, the dot product of the segment's query vector with that page's row of ``y``.

When the profile pass shows that the scores feed nothing but a ``topK`` the launch is deferred
and the ``topK`` runs the fused sm_100a indexer kernel instead (same bits, no score round trip
through HBM).
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import _cabi, _deferred
from ..abs import FORMAT, as_vtensor, vOp, vTensor
from ..abs.tensor import lazy_group_mean_source, materialize
from .context import Context
from ._chain import ChainedOp, tag


class GeMV(vOp):
    _supported = {(FORMAT.BATCHED, FORMAT.PAGED): FORMAT.RAGGED}

    def __init__(self):
        super().__init__()
        self.impl = None
        self.output_format: Optional[FORMAT] = None
        self.output_buffer: Optional[torch.Tensor] = None
        # fusion bookkeeping (see output_func.topK.profile)
        self._x_is_group_mean = False
        self._score_read_elsewhere = False
        self._fused_consumer = None
        self._pending = None

    def profile(self, x: vTensor, y: vTensor, ctx: Context) -> vTensor:
        p = self._prefix()
        assert isinstance(x, vTensor), f"{p}profile expects x to be vTensor, got {type(x)}"
        assert isinstance(y, vTensor), f"{p}profile expects y to be vTensor, got {type(y)}"
        assert x.dim() == 3 and y.dim() == 3, f"{p}expected 3D inputs; got x.ndim={x.dim()}, y.ndim={y.dim()}"
        assert x.shape[1] == 1, f"{p}expected x.shape[1] == 1, got {tuple(x.shape)}"
        assert y.shape[1] == 1, f"{p}expected y.shape[1] == 1, got {tuple(y.shape)}"
        assert x.shape[2] == y.shape[2], (
            f"{p}last dimension mismatch: x.shape[2]={x.shape[2]} vs y.shape[2]={y.shape[2]}")
        key = (x._format, y._format)
        assert key in self._supported, (
            f"{p}no implementation for (x_fmt={x._format}, y_fmt={y._format}). "
            f"Available: {list(self._supported)}")
        self.impl = _cabi.gemv
        self.output_format = self._supported[key]
        self.output_buffer = torch.empty((ctx.max_num_pages, 1, 1), device=x.device, dtype=x.dtype)
        ctx.add_aux_memory(self.output_buffer)
        ctx.add_aux_flops(y.shape[1] * y.shape[2])  # one multiply-add row per page of the PAGED operand
        self._x_is_group_mean = getattr(x, "_vtx_origin", None) == "group_mean"
        out = as_vtensor(self.output_buffer, self.output_format)
        out._vtx_producer = self
        return out

    def execute(self, x: torch.Tensor, y: torch.Tensor, ctx: Context) -> torch.Tensor:
        p = self._prefix()
        assert self.impl is not None, f"{p}execute called before profile() (impl is None)"
        assert x.device == y.device == self.output_buffer.device, (
            f"{p}device mismatch: x={x.device}, y={y.device}, o={self.output_buffer.device}")
        if self._fused_consumer is not None and not self._score_read_elsewhere:
            src = lazy_group_mean_source(x)
            self._pending = (src if src is not None else x, y)
            return self.output_buffer
        x = materialize(x)
        _deferred.flush_all()  # eager launch: anything recorded earlier must reach the GPU first
        eff_bs = ctx.batch_size * ctx.num_kv_heads
        self.impl(x, y, self.output_buffer, ctx.dense_kv_indptr, ctx.dense_kv_indices, eff_bs, ctx.topk_val,
                  ctx.page_reserved_bos, ctx.page_reserved_eos)
        return self.output_buffer


class GeMM(vOp, ChainedOp):
    """``GeMM()(x, y, ctx=ctx)`` computes ``O[p] = Y[row_p] X[s]^T`` per candidate page (reference:
    ``indexer/matmul.py:194-399`` over ``mm_bpr``): ``x`` BATCHED ``[S, G, D]``, ``y`` PAGED ``[num_pages*H, C, D]`` ->
    RAGGED ``[max_num_pages, C, G]`` (fp32 products and sum, rounded once to the input dtype).

    Kernel: ``vtx_gemm_bpr``; with ``C == 1`` it is also the head of the fused chain
    ``GeMM -> Softmax -> Max -> topK``.  The RAGGED-operand forms of the reference (``mm_rrr``, ``mm_rpr``) are
    not built.
    """

    def __init__(self):
        super().__init__()
        self.output_buffer: Optional[torch.Tensor] = None
        self.output_format: Optional[FORMAT] = None
        self._pending = None

    def profile(self, x: vTensor, y: vTensor, ctx: Context) -> vTensor:
        p = self._prefix()
        assert isinstance(x, vTensor) and isinstance(y, vTensor), f"{p}profile expects vTensor inputs"
        assert x.dim() == 3 and y.dim() == 3, f"{p}expected 3D inputs; got x.ndim={x.dim()}, y.ndim={y.dim()}"
        assert x.shape[2] == y.shape[2], f"{p}last dimension mismatch: {x.shape[2]} vs {y.shape[2]}"
        key = (x._format, y._format)
        if key != (FORMAT.BATCHED, FORMAT.PAGED):
            raise NotImplementedError(f"{p}only (BATCHED, PAGED) operands have an sm_100a kernel; got {key}")
        if x.dtype != torch.bfloat16 or y.dtype != torch.bfloat16:
            raise NotImplementedError(f"{p}the GeMM kernel is built for bfloat16")
        self.output_format = FORMAT.RAGGED
        self.output_buffer = torch.empty((ctx.max_num_pages, y.shape[1], x.shape[1]), device=x.device, dtype=x.dtype)
        ctx.add_aux_memory(self.output_buffer)
        ctx.add_aux_flops(x.shape[1] * y.shape[1] * y.shape[2])
        out = as_vtensor(self.output_buffer, self.output_format)
        tag(out, [("gemm", self)], self)
        return out

    def execute(self, x: torch.Tensor, y: torch.Tensor, ctx: Context) -> torch.Tensor:
        assert self.output_buffer is not None, f"{self._prefix()}execute called before profile()"
        x = materialize(x)
        if self._runs_fused():
            self._pending = (x, y)  # the chain's last operator launches the fused kernel
            return self.output_buffer
        _deferred.flush_all()
        ptr, eff, K, bos, eos = _cabi._win(ctx)
        _cabi.gemm_bpr(x, y, self.output_buffer, ptr, ctx.dense_kv_indices, eff, K, bos, eos)
        return self.output_buffer
