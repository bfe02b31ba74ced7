"""Unary elementwise operators of the indexer (reference: ``indexer/elementwise.py:8-297``).

``Relu``, ``Sigmoid``, ``Silu``, ``Abs`` and ``Add_Mul`` take a RAGGED tensor ``[S, C, D]`` (for example the
scores a ``GeMV`` returns) and return a RAGGED tensor of the same shape held by the operator:

* ``Relu(alpha, beta)``:     ``x >= alpha ? x : beta``
* ``Sigmoid(alpha, beta)``:  ``1 / (1 + exp(beta * x + alpha))``
* ``Silu(alpha, beta)``:     ``x / (1 + exp(beta * x + alpha))``
* ``Abs(alpha, beta)``:      ``|beta * x + alpha|``
* ``Add_Mul(alpha, beta)``:  ``beta * x + alpha``

One sm_100a kernel (``vtx_elementwise``) serves all five; it processes the packed rows
``[0, dense_kv_indptr[batch_size * num_kv_heads])``, the union of the reference's workload windows.
bf16 only, as in the reference kernel.
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import _cabi, _deferred
from ..abs import FORMAT, as_vtensor, vOp, vTensor
from ..utils import ElementwiseOpType
from .context import Context


class Elementwise(vOp):
    _supported = {FORMAT.RAGGED: FORMAT.RAGGED}

    def __init__(self, alpha: float = 1.0, beta: float = 1.0):
        super().__init__()
        self.impl = None
        self.op_type: Optional[ElementwiseOpType] = None
        self.alpha = alpha
        self.beta = beta
        self.output_format: Optional[FORMAT] = None
        self.output_buffer: Optional[torch.Tensor] = None

    def profile(self, x: vTensor, ctx: Context) -> vTensor:
        p = self._prefix()
        assert isinstance(x, vTensor), f"{p}profile expects x to be vTensor, got {type(x)}"
        assert x.dim() == 3, f"{p}expected 3D input [S, C, D]. Got ndim={x.dim()} shape={tuple(x.shape)}"
        assert x._format in self._supported, (
            f"{p}no implementation for x_fmt={x._format}. Available keys: {list(self._supported)}")
        if x.dtype != torch.bfloat16:
            raise NotImplementedError(f"{p}the elementwise kernel is built for bfloat16, got {x.dtype}")
        self.impl = _cabi.elementwise
        self.output_format = self._supported[x._format]
        self.output_buffer = torch.empty((ctx.max_num_pages, x.shape[1], x.shape[2]), device=x.device, dtype=x.dtype)
        ctx.add_aux_memory(self.output_buffer)
        producer = getattr(x, "_vtx_producer", None)
        if producer is not None and hasattr(producer, "_score_read_elsewhere"):
            producer._score_read_elsewhere = True  # its scores must really be written: no fusion into topK
        return as_vtensor(self.output_buffer, self.output_format)

    def execute(self, x: torch.Tensor, ctx: Context) -> torch.Tensor:
        p = self._prefix()
        assert self.impl is not None, f"{p}execute called before profile() (impl is None)"
        assert self.output_buffer is not None, f"{p}output buffer is None; did profile() run?"
        assert x.device == self.output_buffer.device, (
            f"{p}device mismatch: x.device={x.device}, o.device={self.output_buffer.device}")
        _deferred.flush_all()  # eager launch: anything recorded earlier must reach the GPU first
        eff_bs = ctx.batch_size * ctx.num_kv_heads
        self.impl(x, self.output_buffer, ctx.dense_kv_indptr[eff_bs:eff_bs + 1], self.op_type.value, self.alpha,
                  self.beta)
        return self.output_buffer


class Relu(Elementwise):
    def __init__(self, alpha: float = 0.0, beta: float = 0.0):
        super().__init__(alpha, beta)
        self.op_type = ElementwiseOpType.Relu


class Silu(Elementwise):
    def __init__(self, alpha: float = 0.0, beta: float = 0.0):
        super().__init__(alpha, beta)
        self.op_type = ElementwiseOpType.Silu


class Sigmoid(Elementwise):
    def __init__(self, alpha: float = 0.0, beta: float = 0.0):
        super().__init__(alpha, beta)
        self.op_type = ElementwiseOpType.Sigmoid


class Add_Mul(Elementwise):
    def __init__(self, alpha: float = 0.0, beta: float = 1.0):
        super().__init__(alpha, beta)
        self.op_type = ElementwiseOpType.Add_Mul


class Abs(Elementwise):
    def __init__(self, alpha: float = 0.0, beta: float = 1.0):
        super().__init__(alpha, beta)
        self.op_type = ElementwiseOpType.Abs
