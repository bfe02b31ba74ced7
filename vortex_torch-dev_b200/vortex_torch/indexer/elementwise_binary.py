"""Elementwise binary operators (reference: ``indexer/elementwise_binary.py``).

``Multiply()(x, y, ctx=ctx)`` with ``x`` BATCHED ``[S, G, D]`` and ``y`` PAGED ``[num_pages*H, 1, D]`` gives the
RAGGED ``[S_pack, G, D]`` products (rounded to the input dtype); ``Maximum()(a, b, ctx=ctx)`` is the
elementwise maximum of two RAGGED tensors.  On sm_100a both exist as links of the fused chain of the
``gqa_quest_sparse_attention`` indexer (``Multiply x2 -> Maximum -> Sum(dim=2) -> Max(dim=1) -> topK``).
"""
from __future__ import annotations

from typing import Optional

import torch

from ..abs import FORMAT, as_vtensor, vOp, vTensor
from ..abs.tensor import materialize
from ._chain import ChainedOp, tag
from ._unbuilt import unbuilt
from .context import Context


class Multiply(vOp, ChainedOp):
    def __init__(self):
        super().__init__()
        self.output_buffer: Optional[torch.Tensor] = None
        self._pending = None

    def profile(self, x: vTensor, y: vTensor, ctx: Context) -> vTensor:
        p = self._prefix()
        assert isinstance(x, vTensor) and isinstance(y, vTensor), f"{p}profile expects vTensor inputs"
        assert x.dim() == 3 and y.dim() == 3, f"{p}expected 3D inputs"
        if (x._format, y._format) != (FORMAT.BATCHED, FORMAT.PAGED):
            raise NotImplementedError(f"{p}only (BATCHED, PAGED) inputs are built; got ({x._format}, {y._format})")
        assert x.shape[2] == y.shape[2], f"{p}last dimension mismatch: {x.shape[2]} vs {y.shape[2]}"
        d0 = max(x.shape[1], y.shape[1])
        self.output_buffer = torch.empty((ctx.max_num_pages, d0, x.shape[2]), device=x.device, dtype=x.dtype)
        ctx.add_aux_memory(self.output_buffer)
        ctx.add_aux_flops(d0 * x.shape[2])
        out = as_vtensor(self.output_buffer, FORMAT.RAGGED)
        tag(out, [("multiply", self)], self)
        self._y_rows = y.shape[1]
        return out

    def execute(self, x: torch.Tensor, y: torch.Tensor, ctx: Context) -> torch.Tensor:
        self._require_fused("Multiply")
        self._pending = (materialize(x), y)
        return self.output_buffer


class Maximum(vOp, ChainedOp):
    def __init__(self):
        super().__init__()
        self.output_buffer: Optional[torch.Tensor] = None

    def profile(self, x: vTensor, y: vTensor, ctx: Context) -> vTensor:
        p = self._prefix()
        assert isinstance(x, vTensor) and isinstance(y, vTensor), f"{p}profile expects vTensor inputs"
        assert x.shape == y.shape, f"{p}shape mismatch: {tuple(x.shape)} vs {tuple(y.shape)}"
        if (x._format, y._format) != (FORMAT.RAGGED, FORMAT.RAGGED):
            raise NotImplementedError(f"{p}only (RAGGED, RAGGED) inputs are built")
        self.output_buffer = torch.empty(tuple(x.shape), device=x.device, dtype=x.dtype)
        ctx.add_aux_memory(self.output_buffer)
        out = as_vtensor(self.output_buffer, FORMAT.RAGGED)
        srcs = [getattr(t, "_vtx_chain", []) for t in (x, y)]
        tag(out, [("maximum", self, srcs)], self)
        return out

    def execute(self, x: torch.Tensor, y: torch.Tensor, ctx: Context) -> torch.Tensor:
        self._require_fused("Maximum")
        return self.output_buffer


class _RaggedBinary(vOp):
    """Stand-alone binary operator on two RAGGED tensors (``vtx_elementwise_binary``): both inputs are real
    buffers (for example the scores of two ``GeMV`` operators), the result is a RAGGED tensor held by the
    operator.  Inner dims broadcast as in the reference (``indexer/elementwise_binary.py:115-128``)."""

    _op_code = -1

    def __init__(self, alpha: float = 1.0, beta: float = 1.0):
        super().__init__()
        self.alpha, self.beta = alpha, beta
        self.output_format: Optional[FORMAT] = None
        self.output_buffer: Optional[torch.Tensor] = None

    def profile(self, x: vTensor, y: vTensor, ctx: Context) -> vTensor:
        p = self._prefix()
        assert isinstance(x, vTensor), f"{p}profile expects x to be vTensor, got {type(x)}"
        assert isinstance(y, vTensor), f"{p}profile expects y to be vTensor, got {type(y)}"
        assert x.dim() == 3 and y.dim() == 3, f"{p}expected 3D inputs [S, C, D]; got x.ndim={x.dim()}, y.ndim={y.dim()}"
        assert x.shape[1] == y.shape[1] or x.shape[1] == 1 or y.shape[1] == 1, (
            f"{p}dim-1 not broadcastable: x.shape={tuple(x.shape)}, y.shape={tuple(y.shape)}")
        assert x.shape[2] == y.shape[2] or x.shape[2] == 1 or y.shape[2] == 1, (
            f"{p}dim-2 not broadcastable: x.shape={tuple(x.shape)}, y.shape={tuple(y.shape)}")
        if (x._format, y._format) != (FORMAT.RAGGED, FORMAT.RAGGED):
            raise NotImplementedError(f"{p}only (RAGGED, RAGGED) inputs are built; got ({x._format}, {y._format})")
        if x.dtype != torch.bfloat16 or y.dtype != torch.bfloat16:
            raise NotImplementedError(f"{p}the elementwise kernels are built for bfloat16")
        for t in (x, y):
            producer = getattr(t, "_vtx_producer", None)
            if producer is not None and hasattr(producer, "_score_read_elsewhere"):
                producer._score_read_elsewhere = True  # its output must really be written
        self.output_format = FORMAT.RAGGED
        self.output_buffer = torch.empty((ctx.max_num_pages, max(x.shape[1], y.shape[1]), max(x.shape[2], y.shape[2])),
                                         device=x.device, dtype=x.dtype)
        ctx.add_aux_memory(self.output_buffer)
        return as_vtensor(self.output_buffer, self.output_format)

    def execute(self, x: torch.Tensor, y: torch.Tensor, ctx: Context) -> torch.Tensor:
        from .. import _cabi, _deferred

        assert self.output_buffer is not None, f"{self._prefix()}execute called before profile()"
        _deferred.flush_all()
        eff_bs = ctx.batch_size * ctx.num_kv_heads
        _cabi.elementwise_binary(materialize(x), materialize(y), self.output_buffer,
                                 ctx.dense_kv_indptr[eff_bs:eff_bs + 1], self._op_code, self.alpha, self.beta)
        return self.output_buffer


class Minimum(_RaggedBinary):
    _op_code = 1


class Add(_RaggedBinary):
    """``alpha * x + beta * y`` (each product and the sum rounded once to bf16)."""

    _op_code = 2
