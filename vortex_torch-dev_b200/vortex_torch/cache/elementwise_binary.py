"""Cache-side binary elementwise operators (reference: ``cache/elementwise_binary.py:8-519``).

``Maximum / Minimum / Add / Multiply (alpha, beta)(x, y, output, loc=loc, ctx=ctx)``: for every new token slot in
``loc`` that closes a page, and every KV head, combine that page's blocks of ``x`` and ``y`` (inner dims of size 1
repeat) into the block of ``output``.  ``x`` and ``y`` share a layout, PAGED or RAGGED, and ``output`` has either
(reference kernels ``elementwise_binary_ppp / _ppr / _rrp / _rrr``); without ``output`` the operator owns a
RAGGED buffer.  Kernel: ``vtx_cache_binary``.
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import _cabi, _deferred
from ..abs import FORMAT, vOp, vTensor
from ..utils import ElementwiseBinaryOpType
from ._common import check_operand, resolve_output
from .context import Context


class Elementwise_Binary(vOp):
    op_type: Optional[ElementwiseBinaryOpType] = None

    def __init__(self, alpha: float = 1.0, beta: float = 1.0):
        super().__init__()
        self.alpha, self.beta = alpha, beta
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
        assert x.shape[1] == y.shape[1] or x.shape[1] == 1 or y.shape[1] == 1, (
            f"{p}dim-1 not broadcastable: x.shape={tuple(x.shape)}, y.shape={tuple(y.shape)}")
        assert x.shape[2] == y.shape[2] or x.shape[2] == 1 or y.shape[2] == 1, (
            f"{p}dim-2 not broadcastable: x.shape={tuple(x.shape)}, y.shape={tuple(y.shape)}")
        inner = (max(x.shape[1], y.shape[1]), max(x.shape[2], y.shape[2]))
        out, self.output_buffer = resolve_output(p, x, output, inner, ctx)
        self.output_format = out._format
        self._layout = (x._format == FORMAT.RAGGED, out._format == FORMAT.RAGGED)
        ctx.add_aux_flops(inner[0] * inner[1])
        return out

    def execute(self, x: torch.Tensor, y: torch.Tensor, output: Optional[torch.Tensor], loc: torch.Tensor,
                ctx: Context) -> torch.Tensor:
        assert self._layout is not None, f"{self._prefix()}called before profile()"
        out = self.output_buffer if output is None else output
        _deferred.flush_all()
        ctx.flush_kv_write()
        _cabi.cache_binary(x, y, out, loc, ctx.head_num, ctx.page_size, self.op_type.value, self.alpha, self.beta,
                           in_ragged=self._layout[0], out_ragged=self._layout[1])
        return out


class Maximum(Elementwise_Binary):
    op_type = ElementwiseBinaryOpType.Maximum


class Minimum(Elementwise_Binary):
    op_type = ElementwiseBinaryOpType.Minimum


class Add(Elementwise_Binary):
    op_type = ElementwiseBinaryOpType.Add


class Multiply(Elementwise_Binary):
    op_type = ElementwiseBinaryOpType.Mul
