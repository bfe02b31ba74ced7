"""Page-completion reductions (reference ops: ``cache/reduce.py:10-525``).

``Mean(dim=1)(x, output, loc=loc, ctx=ctx)`` — the ``CMean`` of the shipped flows: for every new
token slot in ``loc`` that closes a page, and every KV head, reduce that page's block of ``x``
(``[rows, cols]``) over its rows and write ``output[row, 0, :]``.  Accumulation is fp32 in row
order with one rounding to the cache dtype.  ``Mean / Max / Min / L2Norm`` with ``dim`` 1 or 2 and ``x`` / ``output``
PAGED or RAGGED in any combination are built (reference kernels ``reduce_pp / _rp / _pr / _rr``); without
``output`` the operator owns a RAGGED buffer.  PAGED -> PAGED ``Mean / Max / Min (dim=1)`` take the tuned kernel
(``vtx_creduce``) that the runtime can also fold into its KV write and attention launches; everything else
goes through ``vtx_cache_reduce``.
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import _cabi
from ..abs import FORMAT, vOp, vTensor
from ..utils import ReduceType
from .context import Context


class Reduce(vOp):
    def __init__(self, dim: int = 1):
        super().__init__()
        assert dim in (1, 2), f"{type(self).__name__}.__init__: dim must be 1 or 2, got dim={dim}"
        self.dim = dim
        self.reduce_type: Optional[ReduceType] = None
        self.impl = None
        self.output_format: Optional[FORMAT] = None
        self.output_buffer: Optional[torch.Tensor] = None

    def profile(self, x: vTensor, output: Optional[vTensor], loc: torch.Tensor, ctx: Context) -> vTensor:
        from ._common import check_operand, resolve_output

        p = self._prefix()
        assert isinstance(x, vTensor), f"{p}x must be vTensor, got {type(x)}"
        assert isinstance(loc, torch.Tensor), f"{p}loc must be torch.Tensor, got {type(loc)}"
        assert x.dim() == 3, f"{p}x must be 3D, got ndim={x.dim()} shape={tuple(x.shape)}"
        inner = (1, x.shape[2]) if self.dim == 1 else (x.shape[1], 1)
        fast = (output is not None and isinstance(output, vTensor) and (x._format, output._format) == (FORMAT.PAGED, FORMAT.PAGED)
                and self.dim == 1 and self.reduce_type in (ReduceType.Mean, ReduceType.Max, ReduceType.Min))
        if fast:
            assert output.dim() == 3, f"{p}output must be 3D, got ndim={output.dim()} shape={tuple(output.shape)}"
            assert output.shape[1] == 1, f"{p}profile(dim=1): expected output.shape[1] == 1, got {tuple(output.shape)}"
            assert output.shape[2] == x.shape[2], (
                f"{p}profile(dim=1): expected output.shape[2] == x.shape[2], got {output.shape[2]} vs {x.shape[2]}")
            assert x.device == output.device, (
                f"{p}x and output must be on the same device (x.device={x.device}, output.device={output.device})")
            self.impl = _cabi.cmean
            self.output_format = FORMAT.PAGED
            self._layout = None
            return output
        check_operand(p, "x", x)
        out, self.output_buffer = resolve_output(p, x, output, inner, ctx)
        self.impl = _cabi.cache_reduce
        self.output_format = out._format
        self._layout = (x._format == FORMAT.RAGGED, out._format == FORMAT.RAGGED)
        return out

    def execute(self, x: torch.Tensor, output: Optional[torch.Tensor], loc: torch.Tensor,
                ctx: Context) -> torch.Tensor:
        assert self.impl is not None, f"{self._prefix()}called before profile() (impl is None)"
        if getattr(self, "_layout", None) is not None:  # any layout, any dim, L2Norm: the general kernel
            out = self.output_buffer if output is None else output
            ctx.flush_append()
            ctx.flush_kv_write()
            _cabi.cache_reduce(x, out, loc, ctx.head_num, ctx.page_size, self.dim, self.reduce_type.value,
                               x_ragged=self._layout[0], out_ragged=self._layout[1])
            return out
        from .._deferred import PendingAppend

        pa = getattr(ctx, "_pending_append", None)
        if pa is not None:
            if (pa.kind == "minmax" and pa.summary2 is None and self.reduce_type == ReduceType.Min
                    and pa.write.reduces(x, loc, ctx)):
                pa.summary2 = output  # second half of a recorded "token write + page maximum + page minimum"
                return output
            ctx.flush_append()
        pend = getattr(ctx, "_pending_kv", None)
        if pend is not None:
            defer = pend.pages == "single" and getattr(ctx, "_defer_append", False)
            if self.reduce_type == ReduceType.Mean and pend.reduces(x, loc, ctx):
                # the runtime's KV write and this mean touch the same pages: one kernel does both
                ctx._pending_kv = None
                app = PendingAppend(pend, "mean", output)
                if defer:
                    ctx._pending_append = app  # the caller's attention step may take it along
                else:
                    app.launch(ctx)
                return output
            if self.reduce_type == ReduceType.Max and defer and pend.reduces(x, loc, ctx):
                # the quest flow's cache side: token write + Max now, the Min that follows completes the record
                ctx._pending_kv = None
                ctx._pending_append = PendingAppend(pend, "minmax", output)
                return output
            ctx.flush_kv_write()
        if self.reduce_type == ReduceType.Mean:
            self.impl(x, output, loc, ctx.head_num, ctx.page_size)
        else:
            _cabi.creduce(x, output, loc, ctx.head_num, ctx.page_size, 1 if self.reduce_type == ReduceType.Max else 2)
        return output


class Mean(Reduce):
    def __init__(self, dim: int = 1):
        super().__init__(dim)
        self.reduce_type = ReduceType.Mean


class Max(Reduce):
    def __init__(self, dim: int = 1):
        super().__init__(dim)
        self.reduce_type = ReduceType.Max


class Min(Reduce):
    def __init__(self, dim: int = 1):
        super().__init__(dim)
        self.reduce_type = ReduceType.Min


class L2Norm(Reduce):
    def __init__(self, dim: int = 1):
        super().__init__(dim)
        self.reduce_type = ReduceType.L2Norm
