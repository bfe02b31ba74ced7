"""Scans over the packed page axis (reference: ``indexer/scan.py:8-388``).

``Softmax(dim=0, scale)(x, ctx=ctx)`` replaces, in place, every candidate page's ``[r, c]`` block of the
RAGGED tensor ``x`` by ``softmax(scale * x)`` taken over the candidate pages of its segment (reserved
BOS/EOS pages and segments with no more than ``topk_val`` candidates are left alone), rounded to the
tensor's dtype.  On sm_100a it exists as a link of the fused chain ``GeMM -> Softmax -> Max -> topK``.
"""
from __future__ import annotations

import torch

from ..abs import FORMAT, vOp, vTensor
from ._chain import ChainedOp, chain_of, tag
from ._unbuilt import unbuilt
from .context import Context


class Softmax(vOp, ChainedOp):
    def __init__(self, dim: int = 0, scale: float = 1.0):
        super().__init__()
        assert dim in (0,), f"{self._prefix()}__init__: dim must be 0, got dim={dim}"
        self.dim = dim
        self.scale = scale

    def profile(self, x: vTensor, ctx: Context) -> vTensor:
        p = self._prefix()
        assert isinstance(x, vTensor), f"{p}profile expects x to be vTensor, got {type(x)}"
        assert x.dim() == 3, f"{p}expected x to be 3D, got ndim={x.dim()} shape={tuple(x.shape)}"
        assert x._format == FORMAT.RAGGED, f"{p}no implementation for x._format={x._format}"
        tag(x, chain_of(x) + [("softmax", self)], self)
        return x

    def execute(self, x: torch.Tensor, ctx: Context) -> torch.Tensor:
        self._require_fused("Softmax")
        return x


Normalize = unbuilt("Normalize", "indexer")
