"""Page-completion reductions (reference ops: ``cache/reduce.py:10-525``).

``Mean(dim=1)(x, output, loc=loc, ctx=ctx)`` — the ``CMean`` of the shipped flows: for every new
token slot in ``loc`` that closes a page, and every KV head, reduce that page's block of ``x``
(``[rows, cols]``) over its rows and write ``output[row, 0, :]``.  Accumulation is fp32 in row
order with one rounding to the cache dtype.  Only PAGED -> PAGED with ``dim=1`` has an sm_100a
kernel; other layouts raise ``NotImplementedError`` in the profile pass.
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
        p = self._prefix()
        assert isinstance(x, vTensor), f"{p}x must be vTensor, got {type(x)}"
        assert isinstance(loc, torch.Tensor), f"{p}loc must be torch.Tensor, got {type(loc)}"
        assert x.dim() == 3, f"{p}x must be 3D, got ndim={x.dim()} shape={tuple(x.shape)}"
        if output is None:
            raise NotImplementedError(f"{p}RAGGED-output reductions have no sm_100a kernel in this build")
        assert isinstance(output, vTensor), f"{p}output must be vTensor, got {type(output)}"
        assert output.dim() == 3, f"{p}output must be 3D, got ndim={output.dim()} shape={tuple(output.shape)}"
        if (x._format, output._format) != (FORMAT.PAGED, FORMAT.PAGED) or self.dim != 1 \
                or self.reduce_type not in (ReduceType.Mean, ReduceType.Max, ReduceType.Min):
            raise NotImplementedError(
                f"{p}only Mean/Max/Min(dim=1) PAGED->PAGED have sm_100a kernels; got {self.reduce_type}, "
                f"dim={self.dim}, ({x._format}, {output._format})")
        assert output.shape[1] == 1, f"{p}profile(dim=1): expected output.shape[1] == 1, got {tuple(output.shape)}"
        assert output.shape[2] == x.shape[2], (
            f"{p}profile(dim=1): expected output.shape[2] == x.shape[2], got {output.shape[2]} vs {x.shape[2]}")
        assert x.device == output.device, (
            f"{p}x and output must be on the same device (x.device={x.device}, output.device={output.device})")
        self.impl = _cabi.cmean
        self.output_format = FORMAT.PAGED
        return output

    def execute(self, x: torch.Tensor, output: Optional[torch.Tensor], loc: torch.Tensor,
                ctx: Context) -> torch.Tensor:
        assert self.impl is not None, f"{self._prefix()}called before profile() (impl is None)"
        pa = getattr(ctx, "_pending_append", None)
        if pa is not None:
            if (len(pa) == 8 and pa[5] is None and self.reduce_type == ReduceType.Min
                    and x.data_ptr() == pa[0].data_ptr() and loc.data_ptr() == pa[6].data_ptr()):
                # second half of a recorded "token write + page maximum + page minimum"
                ctx._pending_append = pa[:5] + (output,) + pa[6:]
                return output
            ctx.flush_append()
        pend = getattr(ctx, "_pending_kv", None)
        if pend is not None:
            k_cache, v_cache, new_k, new_v, ploc, P, mode = pend
            single = mode == "single"
            if (mode is not None and self.reduce_type == ReduceType.Mean
                    and x.data_ptr() == k_cache.data_ptr() and loc.data_ptr() == ploc.data_ptr()
                    and loc.shape == ploc.shape and x.shape[1] == P == ctx.page_size
                    and new_k.shape[1] == ctx.head_num):
                # the runtime's KV write and this mean touch the same page: one kernel does both
                ctx._pending_kv = None
                if single and getattr(ctx, "_defer_append", False):
                    ctx.flush_append()
                    ctx._pending_append = (k_cache, v_cache, new_k, new_v, output, loc, P)
                    return output
                _cabi.set_kv_cmean(k_cache, v_cache, new_k, new_v, output, loc, P)
                return output
            if (single and self.reduce_type == ReduceType.Max and getattr(ctx, "_defer_append", False)
                    and x.data_ptr() == k_cache.data_ptr() and loc.data_ptr() == ploc.data_ptr()
                    and loc.shape == ploc.shape and x.shape[1] == P == ctx.page_size
                    and new_k.shape[1] == ctx.head_num):
                # the quest flow's cache side: token write + Max now, the Min that follows completes the record
                ctx._pending_kv = None
                ctx.flush_append()
                ctx._pending_append = (k_cache, v_cache, new_k, new_v, output, None, loc, P)
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
