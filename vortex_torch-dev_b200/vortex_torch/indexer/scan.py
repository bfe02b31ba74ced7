"""Scans over the packed page axis (reference: ``indexer/scan.py:8-388``).

``Softmax(dim=0, scale)(x, ctx=ctx)`` replaces, in place, every candidate page's ``[r, c]`` block of the
RAGGED tensor ``x`` by ``softmax(scale * x)`` taken over the candidate pages of its segment (reserved
BOS/EOS pages and segments with no more than ``topk_val`` candidates are left alone), rounded to the
tensor's dtype.  ``Normalize(dim=0)(x, ctx=ctx)`` divides by the L2 norm over the same axis instead.
Kernels: ``vtx_softmax_ragged`` / ``vtx_normalize_ragged`` (reference: ``softmax_inplace_r_kernel``,
``normalize_inplace_r_kernel``).  ``Softmax`` between ``GeMM`` and ``Max(dim=2)`` is also a link of the fused
indexer kernel of the gqa_block_sparse_attention flow.
"""
from __future__ import annotations

import torch

from .. import _cabi, _deferred
from ..abs import FORMAT, vOp, vTensor
from ._chain import ChainedOp, chain_of, mark_read, note_consumer, tag
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
        assert x._format == FORMAT.RAGGED, f"{p}no implementation for x._format={x._format}. Available: [RAGGED]"
        if x.dtype != torch.bfloat16:
            raise NotImplementedError(f"{p}the softmax kernel is built for bfloat16, got {x.dtype}")
        ctx.add_aux_flops(4 * x.shape[1] * x.shape[2])
        note_consumer(x)
        tag(x, chain_of(x) + [("softmax", self)], self)  # in place: x itself is the output
        return x

    def execute(self, x: torch.Tensor, ctx: Context) -> torch.Tensor:
        if self._runs_fused():
            return x
        _deferred.flush_all()
        _cabi.softmax_ragged(x, *_cabi._win(ctx), self.scale)
        return x


class Normalize(vOp):
    def __init__(self, dim: int = 0):
        super().__init__()
        assert dim in (0,), f"{self._prefix()}__init__: dim must be 0, got dim={dim}"
        self.dim = dim

    def profile(self, x: vTensor, ctx: Context) -> vTensor:
        p = self._prefix()
        assert isinstance(x, vTensor), f"{p}profile expects x to be vTensor, got {type(x)}"
        assert x.dim() == 3, f"{p}expected x to be 3D, got ndim={x.dim()} shape={tuple(x.shape)}"
        assert x._format == FORMAT.RAGGED, f"{p}no implementation for x._format={x._format}. Available: [RAGGED]"
        if x.dtype != torch.bfloat16:
            raise NotImplementedError(f"{p}the normalize kernel is built for bfloat16, got {x.dtype}")
        ctx.add_aux_flops(3 * x.shape[1] * x.shape[2])
        mark_read(x)  # never a link of a fused chain: whatever produced x must really write it
        return x

    def execute(self, x: torch.Tensor, ctx: Context) -> torch.Tensor:
        _deferred.flush_all()
        _cabi.normalize_ragged(x, *_cabi._win(ctx))
        return x
