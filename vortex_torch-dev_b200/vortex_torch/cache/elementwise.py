"""Cache-side unary elementwise operators (reference: ``cache/elementwise.py:8-486``).

``Relu / Silu / Sigmoid / Abs / Add_Mul (alpha, beta)(x, output, loc=loc, ctx=ctx)``: for every new token slot in
``loc`` that closes a page, and every KV head, apply the operator to that page's ``[r, c]`` block of ``x`` and write
the block of ``output`` (same formulas as the indexer-side family).  ``x`` and ``output`` are PAGED or RAGGED in
any combination (reference kernels ``elementwise_pp / _pr / _rp / _rr``); without ``output`` the operator owns
a RAGGED buffer.  Kernel: ``vtx_cache_elementwise``.
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import _cabi, _deferred
from ..abs import FORMAT, vOp, vTensor
from ..utils import ElementwiseOpType
from ._common import check_operand, resolve_output
from .context import Context


class Elementwise(vOp):
    op_type: Optional[ElementwiseOpType] = None

    def __init__(self, alpha: float = 0.0, beta: float = 1.0):
        super().__init__()
        self.alpha, self.beta = alpha, beta
        self.output_format: Optional[FORMAT] = None
        self.output_buffer: Optional[torch.Tensor] = None
        self._layout = None

    def profile(self, x: vTensor, output: Optional[vTensor], loc: torch.Tensor, ctx: Context) -> vTensor:
        p = self._prefix()
        check_operand(p, "x", x)
        assert isinstance(loc, torch.Tensor), f"{p}loc must be torch.Tensor, got {type(loc)}"
        out, self.output_buffer = resolve_output(p, x, output, (x.shape[1], x.shape[2]), ctx)
        self.output_format = out._format
        self._layout = (x._format == FORMAT.RAGGED, out._format == FORMAT.RAGGED)
        ctx.add_aux_flops(x.shape[1] * x.shape[2])
        return out

    def execute(self, x: torch.Tensor, output: Optional[torch.Tensor], loc: torch.Tensor, ctx: Context) -> torch.Tensor:
        assert self._layout is not None, f"{self._prefix()}called before profile()"
        out = self.output_buffer if output is None else output
        _deferred.flush_all()
        ctx.flush_kv_write()
        _cabi.cache_elementwise(x, out, loc, ctx.head_num, ctx.page_size, self.op_type.value, self.alpha, self.beta,
                                x_ragged=self._layout[0], out_ragged=self._layout[1])
        return out


class Relu(Elementwise):
    op_type = ElementwiseOpType.Relu

    def __init__(self, alpha: float = 0.0, beta: float = 0.0):
        super().__init__(alpha, beta)


class Silu(Elementwise):
    op_type = ElementwiseOpType.Silu

    def __init__(self, alpha: float = 0.0, beta: float = 0.0):
        super().__init__(alpha, beta)


class Sigmoid(Elementwise):
    op_type = ElementwiseOpType.Sigmoid

    def __init__(self, alpha: float = 0.0, beta: float = 0.0):
        super().__init__(alpha, beta)


class Add_Mul(Elementwise):
    op_type = ElementwiseOpType.Add_Mul


class Abs(Elementwise):
    op_type = ElementwiseOpType.Abs
