"""Deferred launches: typed records of work that a later call may run as part of one fused kernel.

The runtime may ask a context to record a launch instead of issuing it.  Three kinds of record exist:

* `PendingKVWrite`   - a new-token write handed to the cache context before ``forward_cache`` runs;
* `PendingAppend`    - that write absorbed by the flow's first cache operator (write + page summary);
* `PendingSelection` - the flow's page selection (what its ``topK`` would have launched).

Each record can ``launch()`` itself as stand-alone kernels, and `sparse_layer_launch` runs a selection, an
optional append and the attention over the selected pages as ONE kernel.  Every code path that launches
eagerly and could observe deferred work's results calls ``flush_all()`` first, which issues whatever is
still pending, in registration order.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, List, Optional

import torch

_flushers: List[Callable[[], None]] = []


def register(flush: Callable[[], None]) -> None:
    if flush not in _flushers:
        _flushers.append(flush)


def flush_all() -> None:
    for f in list(_flushers):
        f()


def _same(a: Optional[torch.Tensor], b: Optional[torch.Tensor]) -> bool:
    """Same storage start, shape and dtype (two views of one buffer)."""
    if a is None or b is None:
        return a is b
    return a.data_ptr() == b.data_ptr() and a.shape == b.shape and a.dtype == b.dtype


@dataclass
class PendingKVWrite:
    """``set_kv_buffer_launcher(k_cache, v_cache, new_k, new_v, loc, page_size)`` not yet launched.

    ``pages``: what the caller guarantees about ``loc`` - ``"single"``: no two slots fall into one page (a decode
    step); ``"ordered"``: the rows of one page are consecutive entries in ascending slot order (a prefill);
    ``None``: nothing."""
    k_cache: torch.Tensor
    v_cache: torch.Tensor
    new_k: torch.Tensor
    new_v: torch.Tensor
    loc: torch.Tensor
    page_size: int
    pages: Optional[str] = None

    def launch(self) -> None:
        from . import _cabi

        _cabi.set_kv(self.k_cache, self.v_cache, self.new_k, self.new_v, self.loc, self.page_size)

    def reduces(self, x: torch.Tensor, loc: torch.Tensor, ctx) -> bool:
        """True when a page reduction of ``x`` at ``loc`` covers exactly the pages this write touches."""
        return (self.pages is not None and x.data_ptr() == self.k_cache.data_ptr() and _same(loc, self.loc)
                and x.shape[1] == self.page_size == ctx.page_size and self.new_k.shape[1] == ctx.head_num)


@dataclass
class PendingAppend:
    """A token write together with the summary of the page it closes: ``kind`` ``"mean"`` (summary = centroid
    cache) or ``"minmax"`` (summary = page maximum, summary2 = page minimum; summary2 stays None until the flow's
    Min operator has run)."""
    write: PendingKVWrite
    kind: str
    summary: torch.Tensor
    summary2: Optional[torch.Tensor] = None

    def launch(self, ctx) -> None:
        from . import _cabi

        w = self.write
        if self.kind == "mean":
            _cabi.set_kv_cmean(w.k_cache, w.v_cache, w.new_k, w.new_v, self.summary, w.loc, w.page_size)
            return
        w.launch()
        _cabi.creduce(w.k_cache, self.summary, w.loc, ctx.head_num, ctx.page_size, 1)
        if self.summary2 is not None:
            _cabi.creduce(w.k_cache, self.summary2, w.loc, ctx.head_num, ctx.page_size, 2)


@dataclass
class PendingSelection:
    """A page selection not yet launched.  ``kind``: ``"mean_dot"`` (q.mean -> GeMV -> topK, summary = centroids),
    ``"gqa_softmax"`` (GeMM -> Softmax(scale) -> Max -> topK) or ``"quest"`` (summary = page maximum, summary2 = page
    minimum).  ``out``: the packed sparse page list the selection is written to."""
    kind: str
    q: torch.Tensor
    summary: torch.Tensor
    out: torch.Tensor
    summary2: Optional[torch.Tensor] = None
    softmax_scale: Optional[float] = None

    def launch(self, ctx) -> None:
        from . import _cabi

        eff_bs = ctx.batch_size * ctx.num_kv_heads
        common = (ctx.dense_kv_indptr, ctx.sparse_kv_indptr, ctx.dense_kv_indices, self.out, eff_bs, ctx.topk_val,
                  ctx.page_reserved_bos, ctx.page_reserved_eos, ctx.max_num_pages_per_request)
        if self.kind == "quest":
            _cabi.indexer_quest_fused(self.q, self.summary, self.summary2, *common)
        elif self.kind == "gqa_softmax":
            _cabi.indexer_gqa_softmax_fused(self.q, self.summary, *common, self.softmax_scale)
        else:
            _cabi.indexer_fused(self.q, self.summary, *common)


def sparse_layer_supported(sel: PendingSelection, ctx, k_cache: torch.Tensor) -> bool:
    """Shapes the one-launch layer kernel is built for."""
    return (sel.q.dtype == torch.bfloat16 and k_cache.dtype == torch.bfloat16 and sel.q.dim() == 3
            and sel.q.shape[2] in (64, 128) and sel.q.shape[1] in (1, 2, 4, 8))


def append_joins(app: PendingAppend, sel: PendingSelection, ctx, k_cache, v_cache, page_size: int) -> bool:
    """True when the recorded append can ride in the layer launch of ``sel``: it writes this layer's caches, one
    token per request, and maintains exactly the summaries the selection reads."""
    w = app.write
    if not (w.pages == "single" and _same(w.k_cache, k_cache) and _same(w.v_cache, v_cache)
            and w.page_size == page_size and w.new_k.shape[0] == ctx.batch_size
            and w.new_k.shape[1] == ctx.num_kv_heads and ctx.page_reserved_eos >= 1):
        return False
    if sel.kind == "quest":
        return (app.kind == "minmax" and app.summary2 is not None
                and {app.summary.data_ptr(), app.summary2.data_ptr()} == {sel.summary.data_ptr(), sel.summary2.data_ptr()}
                and app.summary.data_ptr() != app.summary2.data_ptr())
    return app.kind == "mean" and app.summary.data_ptr() == sel.summary.data_ptr()


def sparse_layer_launch(sel: PendingSelection, app: Optional[PendingAppend], ctx, k_cache, v_cache, out,
                        kv_last_page_len, page_size: int, sm_scale: float, workspace=None,
                        early_prologue: bool = False) -> None:
    """Selection ``sel`` [+ append ``app``] + attention over the selected pages into ``out``, one kernel."""
    from . import _cabi

    summary, summary2 = sel.summary, sel.summary2
    nk = nv = loc = None
    if app is not None:
        nk, nv, loc = app.write.new_k, app.write.new_v, app.write.loc
        summary, summary2 = app.summary, app.summary2  # maximum first, minimum second, as the append holds them
    _cabi.sparse_layer_fused(sel.q, summary, k_cache, v_cache, out, ctx.dense_kv_indptr, ctx.sparse_kv_indptr,
                             ctx.dense_kv_indices, sel.out, kv_last_page_len, ctx.batch_size * ctx.num_kv_heads,
                             page_size, ctx.topk_val, ctx.page_reserved_bos, ctx.page_reserved_eos,
                             ctx.max_num_pages_per_request, sm_scale, nk, nv, loc,
                             gqa_softmax_scale=sel.softmax_scale if sel.kind == "gqa_softmax" else None,
                             quest_min=summary2 if sel.kind == "quest" else None, workspace=workspace,
                             early_prologue=early_prologue)
