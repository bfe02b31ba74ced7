"""Elementwise binary operators (reference: ``indexer/elementwise_binary.py:8-326``).

``Maximum / Minimum / Add / Multiply (alpha, beta)(x, y, ctx=ctx)`` with the inner dims broadcast
(a size of 1 repeats).  Three operand layouts, as in the reference:

* ``x`` BATCHED ``[S, a0, a1]``, ``y`` PAGED ``[num_pages*H, b0, b1]``: ``op(x[s], y[row_p])`` for every candidate
  page ``p`` of segment ``s`` (``vtx_binary_bpr``; reference kernel ``elementwise_binary_bpr_kernel``);
* ``x`` RAGGED, ``y`` PAGED: ``op(x[p], y[row_p])`` (same kernel; reference ``elementwise_binary_rpr_kernel``);
* ``x`` RAGGED, ``y`` RAGGED: ``op(x[p], y[p])`` (``vtx_elementwise_binary``; reference
  ``elementwise_binary_rrr_kernel``).

The result is a RAGGED tensor held by the operator.  ``Add`` computes ``alpha * x + beta * y``; every bf16
operation rounds once.  ``Multiply`` on (BATCHED, PAGED) twice, then ``Maximum``, are also links of the fused
indexer kernel of the gqa_quest_sparse_attention flow.
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import _cabi, _deferred
from ..abs import FORMAT, as_vtensor, vOp, vTensor
from ..abs.tensor import materialize
from ..utils import ElementwiseBinaryOpType
from ._chain import ChainedOp, mark_read, note_consumer, tag
from .context import Context

_LAYOUTS = {(FORMAT.BATCHED, FORMAT.PAGED): "bpr", (FORMAT.RAGGED, FORMAT.PAGED): "rpr",
            (FORMAT.RAGGED, FORMAT.RAGGED): "rrr"}


class Elementwise_Binary(vOp, ChainedOp):
    op_type: Optional[ElementwiseBinaryOpType] = None

    def __init__(self, alpha: float = 1.0, beta: float = 1.0):
        super().__init__()
        self.alpha, self.beta = alpha, beta
        self.layout: Optional[str] = None
        self.output_format: Optional[FORMAT] = None
        self.output_buffer: Optional[torch.Tensor] = None
        self._pending = None
        self._y_rows = None

    def profile(self, x: vTensor, y: vTensor, ctx: Context) -> vTensor:
        p = self._prefix()
        assert isinstance(x, vTensor), f"{p}profile expects x to be vTensor, got {type(x)}"
        assert isinstance(y, vTensor), f"{p}profile expects y to be vTensor, got {type(y)}"
        assert x.dim() == 3 and y.dim() == 3, f"{p}expected 3D inputs [S, C, D]; got x.ndim={x.dim()}, y.ndim={y.dim()}"
        assert x.shape[1] == y.shape[1] or x.shape[1] == 1 or y.shape[1] == 1, (
            f"{p}dim-1 not broadcastable: x.shape={tuple(x.shape)}, y.shape={tuple(y.shape)}")
        assert x.shape[2] == y.shape[2] or x.shape[2] == 1 or y.shape[2] == 1, (
            f"{p}dim-2 not broadcastable: x.shape={tuple(x.shape)}, y.shape={tuple(y.shape)}")
        key = (x._format, y._format)
        assert key in _LAYOUTS, f"{p}no implementation for (x_fmt={x._format}, y_fmt={y._format}). Available: {list(_LAYOUTS)}"
        if x.dtype != torch.bfloat16 or y.dtype != torch.bfloat16:
            raise NotImplementedError(f"{p}the elementwise kernels are built for bfloat16")
        self.layout = _LAYOUTS[key]
        self.output_format = FORMAT.RAGGED
        d0, d1 = max(x.shape[1], y.shape[1]), max(x.shape[2], y.shape[2])
        self.output_buffer = torch.empty((ctx.max_num_pages, d0, d1), device=x.device, dtype=x.dtype)
        ctx.add_aux_memory(self.output_buffer)
        ctx.add_aux_flops(d0 * d1)
        out = as_vtensor(self.output_buffer, self.output_format)
        # links of the quest chain: Multiply on (BATCHED, PAGED), then Maximum of two such products
        if self.op_type == ElementwiseBinaryOpType.Mul and self.layout == "bpr":
            self._y_rows = y.shape[1]
            tag(out, [("multiply", self)], self)
        elif self.op_type == ElementwiseBinaryOpType.Maximum and self.layout == "rrr":
            for t in (x, y):
                note_consumer(t)
            tag(out, [("maximum", self, [getattr(t, "_vtx_chain", []) for t in (x, y)])], self)
        else:
            for t in (x, y):
                mark_read(t)
            tag(out, [], self)
        return out

    def execute(self, x: torch.Tensor, y: torch.Tensor, ctx: Context) -> torch.Tensor:
        assert self.output_buffer is not None, f"{self._prefix()}execute called before profile()"
        if self._runs_fused():
            if self.layout == "bpr":
                self._pending = (materialize(x), y)  # the chain's last operator launches the fused kernel
            return self.output_buffer
        _deferred.flush_all()
        x = materialize(x)
        ptr, eff, K, bos, eos = _cabi._win(ctx)
        if self.layout == "rrr":
            _cabi.elementwise_binary(x, materialize(y), self.output_buffer, ctx.dense_kv_indptr[eff:eff + 1],
                                     self.op_type.value, self.alpha, self.beta)
        else:
            _cabi.binary_bpr(x, y, self.output_buffer, ptr, ctx.dense_kv_indices, eff, K, bos, eos, self.op_type.value,
                             self.alpha, self.beta, x_is_ragged=self.layout == "rpr")
        return self.output_buffer


class Maximum(Elementwise_Binary):
    op_type = ElementwiseBinaryOpType.Maximum


class Minimum(Elementwise_Binary):
    op_type = ElementwiseBinaryOpType.Minimum


class Add(Elementwise_Binary):
    """``alpha * x + beta * y`` (each product and the sum rounded once to bf16)."""

    op_type = ElementwiseBinaryOpType.Add


class Multiply(Elementwise_Binary):
    op_type = ElementwiseBinaryOpType.Mul
