"""Cache-side ``GeMM`` (reference: ``cache/matmul.py:9-329``).

``GeMM()(x, y, output, loc=loc, ctx=ctx)``: for every new token slot in ``loc`` that closes a page, and every KV
head, ``O = Y X^T`` of that page's blocks ``X [N_x, K]`` and ``Y [N_y, K]`` -> ``O [N_y, N_x]`` (fp32 products and
sum, one rounding).  ``x`` and ``y`` share a layout, PAGED or RAGGED, ``output`` has either (reference kernels
``gemm_ppp / _ppr / _rrp / _rrr``); without ``output`` the operator owns a RAGGED buffer.  Kernel: ``vtx_cache_gemm``.
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import _cabi, _deferred
from ..abs import FORMAT, vOp, vTensor
from ._common import check_operand, resolve_output
from .context import Context


class GeMM(vOp):
    def __init__(self):
        super().__init__()
        self.output_format: Optional[FORMAT] = None
        self.output_buffer: Optional[torch.Tensor] = None
        self._layout = None

    def profile(self, x: vTensor, y: vTensor, output: Optional[vTensor], loc: torch.Tensor, ctx: Context) -> vTensor:
        p = self._prefix()
        check_operand(p, "x", x)
        check_operand(p, "y", y)
        assert isinstance(loc, torch.Tensor), f"{p}loc must be torch.Tensor, got {type(loc)}"
        assert x._format == y._format, (
            f"{p}no implementation for (x_fmt={x._format}, y_fmt={y._format}): both operands must share a layout")
        assert x.shape[2] == y.shape[2], f"{p}inner dimension mismatch: x.shape[2]={x.shape[2]} vs y.shape[2]={y.shape[2]}"
        out, self.output_buffer = resolve_output(p, x, output, (y.shape[1], x.shape[1]), ctx)
        self.output_format = out._format
        self._layout = (x._format == FORMAT.RAGGED, out._format == FORMAT.RAGGED)
        ctx.add_aux_flops(2 * x.shape[1] * y.shape[1] * x.shape[2])
        return out

    def execute(self, x: torch.Tensor, y: torch.Tensor, output: Optional[torch.Tensor], loc: torch.Tensor,
                ctx: Context) -> torch.Tensor:
        assert self._layout is not None, f"{self._prefix()}called before profile()"
        out = self.output_buffer if output is None else output
        _deferred.flush_all()
        ctx.flush_kv_write()
        _cabi.cache_gemm(x, y, out, loc, ctx.head_num, ctx.page_size, in_ragged=self._layout[0],
                         out_ragged=self._layout[1])
        return out
