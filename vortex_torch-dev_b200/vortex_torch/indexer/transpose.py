"""``Transpose()(x, ctx=ctx)``: swap the two inner dims of every candidate page's block of a RAGGED tensor,
``[S_pack, r, c] -> [S_pack, c, r]`` (reference: ``indexer/transpose.py:7-179`` over ``transpose_rr_kernel``;
kernel here: ``vtx_transpose_ragged``)."""
from __future__ import annotations

from typing import Optional

import torch

from .. import _cabi, _deferred
from ..abs import FORMAT, as_vtensor, vOp, vTensor
from ._chain import mark_read
from .context import Context


class Transpose(vOp):
    def __init__(self):
        super().__init__()
        self.output_format: Optional[FORMAT] = None
        self.output_buffer: Optional[torch.Tensor] = None

    def profile(self, x: vTensor, ctx: Context) -> vTensor:
        p = self._prefix()
        assert isinstance(x, vTensor), f"{p}profile expects x to be vTensor, got {type(x)}"
        assert x.dim() == 3, f"{p}expected 3D x [S, D0, D1], got {tuple(x.shape)}"
        assert x._format == FORMAT.RAGGED, f"{p}no implementation for x_fmt={x._format}. Available keys: [RAGGED]"
        if x.dtype != torch.bfloat16:
            raise NotImplementedError(f"{p}the transpose kernel is built for bfloat16, got {x.dtype}")
        mark_read(x)
        self.output_format = FORMAT.RAGGED
        self.output_buffer = torch.empty((x.shape[0], x.shape[2], x.shape[1]), device=x.device, dtype=x.dtype)
        ctx.add_aux_memory(self.output_buffer)
        return as_vtensor(self.output_buffer, self.output_format)

    def execute(self, x: torch.Tensor, ctx: Context) -> torch.Tensor:
        assert self.output_buffer is not None, f"{self._prefix()}execute called before profile()"
        _deferred.flush_all()
        _cabi.transpose_ragged(x, self.output_buffer, *_cabi._win(ctx))
        return self.output_buffer
