"""``Save`` and ``Load``: move candidate pages' blocks between a RAGGED tensor and a PAGED cache
(reference: ``indexer/save_load.py:7-331`` over ``save_rp_kernel`` / ``load_pr_kernel``; kernel here:
``vtx_save_load_ragged``).

``Save()(x, o, ctx=ctx)``: ``o[row_p] = x[p]`` for every candidate position ``p`` (``x`` RAGGED, ``o`` PAGED with the
same inner dims); returns ``o``.  ``Load()(x, ctx=ctx)``: a RAGGED tensor holding ``x[row_p]`` at position ``p``
(``x`` PAGED)."""
from __future__ import annotations

from typing import Optional

import torch

from .. import _cabi, _deferred
from ..abs import FORMAT, as_vtensor, vOp, vTensor
from ._chain import mark_read
from .context import Context


class Save(vOp):
    def __init__(self):
        super().__init__()
        self.output_format: Optional[FORMAT] = None

    def profile(self, x: vTensor, o: vTensor, ctx: Context) -> vTensor:
        p = self._prefix()
        assert isinstance(x, vTensor), f"{p}profile expects x to be vTensor, got {type(x)}"
        assert isinstance(o, vTensor), f"{p}profile expects o to be vTensor, got {type(o)}"
        assert x.dim() == 3, f"{p}expected 3D x [S, D0, D1], got {tuple(x.shape)}"
        assert o.dim() == 3, f"{p}expected 3D o [S, D0, D1], got {tuple(o.shape)}"
        assert x.shape[1] == o.shape[1], f"{p}expected matching D0: x.shape[1]={x.shape[1]} vs o.shape[1]={o.shape[1]}"
        assert x.shape[2] == o.shape[2], f"{p}expected matching D1: x.shape[2]={x.shape[2]} vs o.shape[2]={o.shape[2]}"
        assert x._format == FORMAT.RAGGED, f"{p}no implementation for x_fmt={x._format}. Available keys: [RAGGED]"
        assert o._format == FORMAT.PAGED, f"{p}output format mismatch. Expected {FORMAT.PAGED}, got {o._format}"
        assert x.device == o.device, f"{p}x and o must be on the same device (x.device={x.device}, o.device={o.device})"
        if x.dtype != torch.bfloat16 or o.dtype != torch.bfloat16:
            raise NotImplementedError(f"{p}the save kernel is built for bfloat16")
        mark_read(x)
        self.output_format = FORMAT.PAGED
        return o

    def execute(self, x: torch.Tensor, o: torch.Tensor, ctx: Context) -> torch.Tensor:
        _deferred.flush_all()
        ptr, eff, K, bos, eos = _cabi._win(ctx)
        _cabi.save_load_ragged(x, o, ptr, ctx.dense_kv_indices, eff, K, bos, eos, save=True)
        return o


class Load(vOp):
    def __init__(self):
        super().__init__()
        self.output_format: Optional[FORMAT] = None
        self.output_buffer: Optional[torch.Tensor] = None

    def profile(self, x: vTensor, ctx: Context) -> vTensor:
        p = self._prefix()
        assert isinstance(x, vTensor), f"{p}profile expects x to be vTensor, got {type(x)}"
        assert x.dim() == 3, f"{p}expected 3D x [S, D0, D1], got {tuple(x.shape)}"
        assert x._format == FORMAT.PAGED, f"{p}no implementation for x_fmt={x._format}. Available keys: [PAGED]"
        if x.dtype != torch.bfloat16:
            raise NotImplementedError(f"{p}the load kernel is built for bfloat16, got {x.dtype}")
        self.output_format = FORMAT.RAGGED
        self.output_buffer = torch.empty((ctx.max_num_pages, x.shape[1], x.shape[2]), device=x.device, dtype=x.dtype)
        ctx.add_aux_memory(self.output_buffer)
        return as_vtensor(self.output_buffer, self.output_format)

    def execute(self, x: torch.Tensor, ctx: Context) -> torch.Tensor:
        assert self.output_buffer is not None, f"{self._prefix()}execute called before profile()"
        _deferred.flush_all()
        ptr, eff, K, bos, eos = _cabi._win(ctx)
        _cabi.save_load_ragged(self.output_buffer, x, ptr, ctx.dense_kv_indices, eff, K, bos, eos, save=False)
        return self.output_buffer
