"""``topK``: complete each segment's sparse page list with its best-scoring pages
(reference op: ``indexer/output_func.py:8-235`` over ``csrc/topk.cu:117-203``).

``topK()(x, o, ctx=ctx)``: ``x`` RAGGED ``[S_pack, 1, 1]`` scores at packed dense positions,
``o`` the packed sparse list (``ctx.sparse_kv_indices``).  For every segment with more than
``topk_val`` candidates the ``topk_val`` best rows (score descending, ties by position) are
written behind the reserved BOS pages.  Returns ``o``.
"""
from __future__ import annotations

import torch

from .. import _cabi, _deferred
from ..abs import FORMAT, vOp, vTensor
from ._chain import chain_of, note_consumer
from .context import Context


class topK(vOp):
    _supported = (FORMAT.RAGGED,)

    def __init__(self):
        super().__init__()
        self.impl = None
        self._fused_producer = None
        self._gqa_chain = None
        self._quest_chain = None

    def profile(self, x: vTensor, o: vTensor, ctx: Context) -> None:
        p = self._prefix()
        assert isinstance(x, vTensor), f"{p}profile expects x to be vTensor, got {type(x)}"
        assert isinstance(o, vTensor), f"{p}profile expects o to be vTensor, got {type(o)}"
        assert x.dim() == 3, f"{p}expected x to be 3D, got ndim={x.dim()} shape={tuple(x.shape)}"
        assert o.dim() == 3, f"{p}expected o to be 3D, got ndim={o.dim()} shape={tuple(o.shape)}"
        assert x.shape[1] == 1 and x.shape[2] == 1, (
            f"{p}expected x.shape[1] == x.shape[2] == 1, got {tuple(x.shape)}")
        assert x._format in self._supported, (
            f"{p}no implementation for x._format={x._format}. Available: {list(self._supported)}")
        assert x.device == o.device, (
            f"{p}x and o must be on the same device (x.device={x.device}, o.device={o.device})")
        self.impl = _cabi.topk
        note_consumer(x)
        # GeMM -> Softmax(dim=0) -> Max(dim=2) -> topK: one fused kernel owned by this operator
        names = [l[0] for l in chain_of(x)]
        if names == ["gemm", "softmax", "max"]:
            gemm, softmax, mx = (l[1] for l in chain_of(x))
            if gemm.output_buffer.shape[1] == 1 and mx.dim == 2:
                self._gqa_chain = (gemm, softmax, mx)
                for op in self._gqa_chain:
                    op._fused_into = self
                return
        # Multiply(q, max) / Multiply(q, min) -> Maximum -> Sum(dim=2) -> Max(dim=1) -> topK: one fused kernel
        links = chain_of(x)
        if [l[0] for l in links] == ["maximum", "sum", "max"]:
            maximum, sum_op, mx = links[0][1], links[1][1], links[2][1]
            srcs = links[0][2]
            if (len(srcs) == 2 and all(len(c) == 1 and c[0][0] == "multiply" for c in srcs)
                    and sum_op.dim == 2 and mx.dim == 1 and all(c[0][1]._y_rows == 1 for c in srcs)):
                mul_a, mul_b = srcs[0][0][1], srcs[1][0][1]
                self._quest_chain = (mul_a, mul_b, maximum, sum_op, mx)
                for op in self._quest_chain:
                    op._fused_into = self
                return
        # Fuse with the producing GeMV when its scores are read by this operator only.
        producer = getattr(x, "_vtx_producer", None)
        if producer is not None and hasattr(producer, "_fused_consumer") and producer._fused_consumer is None:
            producer._fused_consumer = self
            self._fused_producer = producer

    def chain_intact(self) -> bool:
        """True while every link of the chain this operator claimed feeds only the next link."""
        chain = self._quest_chain or self._gqa_chain
        return chain is not None and all(op._link_intact() for op in chain)

    def execute(self, x: torch.Tensor, o: torch.Tensor, ctx: Context) -> torch.Tensor:
        assert self.impl is not None, f"{self._prefix()}execute called before profile() (impl is None)"
        sel = self._fused_selection(x, o)
        if sel is not None:
            ctx.record_or_launch(sel)  # the caller's attention step may run it as part of one layer kernel
            return o
        _deferred.flush_all()  # eager launch: anything recorded earlier must reach the GPU first
        ctx.flush_indexer()
        eff_bs = ctx.batch_size * ctx.num_kv_heads
        self.impl(x, ctx.dense_kv_indptr, ctx.sparse_kv_indptr, ctx.dense_kv_indices, o, eff_bs, ctx.topk_val,
                  ctx.page_reserved_bos, ctx.page_reserved_eos, ctx.max_num_pages_per_request)
        return o

    def _fused_selection(self, x: torch.Tensor, o: torch.Tensor):
        """The chain this operator owns, as one `PendingSelection`, or None when the scores in ``x`` are real."""
        if self._quest_chain is not None and self.chain_intact():
            mul_a, mul_b = self._quest_chain[0], self._quest_chain[1]
            (qa, ya), (qb, yb) = mul_a._pending, mul_b._pending
            mul_a._pending = mul_b._pending = None
            if qa.data_ptr() != qb.data_ptr():
                raise NotImplementedError("topK: the two Multiply operators of the quest chain must share their query")
            return _deferred.PendingSelection("quest", qa, ya, o, summary2=yb)
        if self._gqa_chain is not None and self.chain_intact():
            gemm, softmax, _ = self._gqa_chain
            q, y = gemm._pending
            gemm._pending = None
            return _deferred.PendingSelection("gqa_softmax", q, y, o, softmax_scale=float(softmax.scale))
        prod = self._fused_producer
        if prod is not None and prod._pending is not None and x.data_ptr() == prod.output_buffer.data_ptr():
            q, y = prod._pending
            prod._pending = None
            return _deferred.PendingSelection("mean_dot", q, y, o)
        return None
