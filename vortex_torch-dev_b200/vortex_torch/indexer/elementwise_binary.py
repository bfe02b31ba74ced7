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


Minimum, Add = unbuilt("Minimum", "indexer"), unbuilt("Add", "indexer")
