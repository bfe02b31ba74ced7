"""Per-page reductions of RAGGED tensors (reference: ``indexer/reduce.py:8-438``).

``Max / Min / Mean / L2Norm / Sum (dim)(x, ctx=ctx)`` reduce axis ``dim`` (1 or 2) of every candidate page's
``[r, c]`` block: ``[S_pack, r, c] -> [S_pack, 1, c]`` (dim 1) or ``[S_pack, r, 1]`` (dim 2), fp32 arithmetic,
one rounding to bf16 (``vtx_reduce_ragged``; reference kernel ``reduce_rr_kernel``,
``indexer/triton_kernels/reduce_impl.py:8-120``).  ``Max(dim=2)`` after ``GeMM -> Softmax`` and
``Sum(dim=2) -> Max(dim=1)`` after the quest flow's products are also links of the fused indexer kernels.
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import _cabi, _deferred
from ..abs import FORMAT, as_vtensor, vOp, vTensor
from ..utils import ReduceType
from ._chain import ChainedOp, chain_of, note_consumer, tag
from .context import Context


class Reduce(vOp, ChainedOp):
    _chain_name = "reduce"

    def __init__(self, dim: int = 1):
        super().__init__()
        assert dim in (1, 2), f"{self._prefix()}__init__: dim must be 1 or 2, got dim={dim}"
        self.dim = dim
        self.reduce_type: Optional[ReduceType] = None
        self.output_format: Optional[FORMAT] = None
        self.output_buffer: Optional[torch.Tensor] = None

    def profile(self, x: vTensor, ctx: Context) -> vTensor:
        p = self._prefix()
        assert isinstance(x, vTensor), f"{p}profile expects x to be vTensor, got {type(x)}"
        assert x.dim() == 3, f"{p}expected x to be 3D, got ndim={x.dim()} shape={tuple(x.shape)}"
        assert x._format == FORMAT.RAGGED, f"{p}no implementation for x._format={x._format}. Available: [RAGGED]"
        if x.dtype != torch.bfloat16:
            raise NotImplementedError(f"{p}the RAGGED reduction kernel is built for bfloat16, got {x.dtype}")
        d0 = 1 if self.dim == 1 else x.shape[1]
        d1 = 1 if self.dim == 2 else x.shape[2]
        self.output_format = FORMAT.RAGGED
        self.output_buffer = torch.empty((x.shape[0], d0, d1), device=x.device, dtype=x.dtype)
        ctx.add_aux_memory(self.output_buffer)
        ctx.add_aux_flops(x.shape[1] * x.shape[2])
        note_consumer(x)
        out = as_vtensor(self.output_buffer, FORMAT.RAGGED)
        tag(out, chain_of(x) + [(self._chain_name, self)], self)
        return out

    def execute(self, x: torch.Tensor, ctx: Context) -> torch.Tensor:
        assert self.output_buffer is not None, f"{self._prefix()}execute called before profile()"
        if self._runs_fused():
            return self.output_buffer  # the chain's last operator launches the fused kernel
        _deferred.flush_all()
        _cabi.reduce_ragged(x, self.output_buffer, self.dim, self.reduce_type.value, *_cabi._win(ctx))
        return self.output_buffer


class Max(Reduce):
    _chain_name = "max"

    def __init__(self, dim: int = 1):
        super().__init__(dim)
        self.reduce_type = ReduceType.Max


class Min(Reduce):
    _chain_name = "min"

    def __init__(self, dim: int = 1):
        super().__init__(dim)
        self.reduce_type = ReduceType.Min


class Mean(Reduce):
    _chain_name = "mean"

    def __init__(self, dim: int = 1):
        super().__init__(dim)
        self.reduce_type = ReduceType.Mean


class L2Norm(Reduce):
    _chain_name = "l2norm"

    def __init__(self, dim: int = 1):
        super().__init__(dim)
        self.reduce_type = ReduceType.L2Norm


class Sum(Reduce):
    _chain_name = "sum"

    def __init__(self, dim: int = 1):
        super().__init__(dim)
        self.reduce_type = ReduceType.Sum
