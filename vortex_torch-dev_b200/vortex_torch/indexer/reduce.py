"""Per-page reductions of RAGGED tensors (reference: ``indexer/reduce.py:165-309``).

``Max(dim=2)(x, ctx=ctx)`` reduces the last axis of every page block, ``[S_pack, r, c] -> [S_pack, r, 1]``.
On sm_100a ``Max(dim=2)`` exists as a link of the fused chain ``GeMM -> Softmax -> Max -> topK``; the other
reductions are placeholders, except ``Sum(dim=2)`` and ``Max(dim=1)`` which are links of the quest
indexer's fused chain.
"""
from __future__ import annotations

from typing import Optional

import torch

from ..abs import FORMAT, as_vtensor, vOp, vTensor
from ..utils import ReduceType
from ._chain import ChainedOp, chain_of, tag
from ._unbuilt import unbuilt
from .context import Context


class Max(vOp, ChainedOp):
    def __init__(self, dim: int = 1):
        super().__init__()
        assert dim in (1, 2), f"{self._prefix()}__init__: dim must be 1 or 2, got dim={dim}"
        self.dim = dim
        self.reduce_type = ReduceType.Max
        self.output_buffer: Optional[torch.Tensor] = None

    def profile(self, x: vTensor, ctx: Context) -> vTensor:
        p = self._prefix()
        assert isinstance(x, vTensor), f"{p}profile expects x to be vTensor, got {type(x)}"
        assert x.dim() == 3, f"{p}expected x to be 3D, got ndim={x.dim()} shape={tuple(x.shape)}"
        assert x._format == FORMAT.RAGGED, f"{p}no implementation for x._format={x._format}"
        d0 = 1 if self.dim == 1 else x.shape[1]
        d1 = 1 if self.dim == 2 else x.shape[2]
        self.output_buffer = torch.empty((x.shape[0], d0, d1), device=x.device, dtype=x.dtype)
        ctx.add_aux_memory(self.output_buffer)
        out = as_vtensor(self.output_buffer, FORMAT.RAGGED)
        tag(out, chain_of(x) + [("max", self)], self)
        return out

    def execute(self, x: torch.Tensor, ctx: Context) -> torch.Tensor:
        self._require_fused("Max")
        return self.output_buffer


class Sum(Max):
    """``Sum(dim=2)``: fp32 sum over the last axis, rounded once (a link of the quest indexer's fused chain)."""

    def __init__(self, dim: int = 1):
        super().__init__(dim)
        self.reduce_type = ReduceType.Sum

    def profile(self, x: vTensor, ctx: Context) -> vTensor:
        out = super().profile(x, ctx)
        out._vtx_chain[-1] = ("sum", self)
        return out

    def execute(self, x: torch.Tensor, ctx: Context) -> torch.Tensor:
        self._require_fused("Sum")
        return self.output_buffer


Mean, Min, L2Norm = (unbuilt(n, "indexer") for n in ("Mean", "Min", "L2Norm"))
