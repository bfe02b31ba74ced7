"""In-place page fill (reference: ``cache/fill.py:8-165``, kernel ``fill_p_kernel`` of
``cache/triton_kernels/fill_impl.py:6-49``).

``Fill(alpha)(x, loc=loc, ctx=ctx)``: for every new token slot in ``loc`` that closes a page, and every KV head,
overwrite that page's whole ``[D0, D1]`` block of the PAGED tensor ``x`` with ``alpha`` (rounded to bf16).  Nothing
else of ``x`` is touched and ``x`` itself is returned.  The reference does not list the operator in its package
exports; it is importable as ``vortex_torch.cache.fill.Fill`` there and here.  Kernel: ``vtx_cache_elementwise``
with its fill code.
"""
from __future__ import annotations

import torch

from .. import _cabi, _deferred
from ..abs import FORMAT, vOp, vTensor
from .context import Context

_FILL = 5  # op code of vtx_cache_elementwise: write alpha, read nothing


class Fill(vOp):
    def __init__(self, alpha: float = 0.0):
        super().__init__()
        self.alpha = alpha
        self.impl = None

    def profile(self, x: vTensor, loc: torch.Tensor, ctx: Context) -> vTensor:
        p = self._prefix()
        assert isinstance(x, vTensor), f"{p}profile expects x to be vTensor, got {type(x)}"
        assert isinstance(loc, torch.Tensor), f"{p}profile expects loc to be torch.Tensor, got {type(loc)}"
        assert x.dim() == 3, f"{p}expected 3D input [B, D0, D1], got ndim={x.dim()} shape={tuple(x.shape)}"
        assert x._format == FORMAT.PAGED, f"{p}no implementation for x_fmt={x._format}. Available keys: [FORMAT.PAGED]"
        self.impl = _cabi.cache_elementwise
        return x

    def execute(self, x: torch.Tensor, loc: torch.Tensor, ctx: Context) -> torch.Tensor:
        assert self.impl is not None, f"{self._prefix()}called before profile() (impl is None)"
        _deferred.flush_all()
        ctx.flush_kv_write()
        self.impl(x, x, loc, ctx.head_num, ctx.page_size, _FILL, self.alpha, 0.0)
        return x
