"""``vFlow``: the contract a sparse-attention algorithm implements.

A flow supplies three methods (reference: ``flow/flow.py:171-326``):

``forward_indexer(q, o, cache, ctx)``
    called once per sparse layer per decode step.  ``q`` is ``[bs*H_kv, G, D]`` (BATCHED),
    ``o`` is the packed sparse page list viewed ``[S_sparse, 1, 1]`` (RAGGED) that ``topK``
    completes in place, ``cache[name]`` are per-layer page summaries ``[num_pages*H_kv, r, c]``
    (PAGED).  Only ``q`` may be touched with plain torch ops.
``forward_cache(cache, loc, ctx)``
    called after new K/V tokens were written; ``loc`` holds their cache slots.  Cache
    operators do work only for slots that complete a page, so each page is summarised once.
``create_cache(page_size, head_dim)``
    returns ``{name: (rows, cols)}`` for the extra per-page caches the flow needs.

The remaining methods are helpers the serving runtime calls (``flow/flow.py:331-460``).
"""
from __future__ import annotations

from abc import ABC, abstractmethod
from typing import Dict, Tuple

import torch

from ..abs import ContextBase

CacheShapes = Dict[str, Tuple[int, int]]


class vFlow(ABC):
    def __init__(self):
        super().__init__()

    @abstractmethod
    def forward_indexer(self, q: torch.Tensor, o: torch.Tensor, cache: Dict[str, torch.Tensor],
                        ctx: ContextBase):
        ...

    @abstractmethod
    def forward_cache(self, cache: Dict[str, torch.Tensor], loc: torch.Tensor, ctx: ContextBase):
        ...

    @abstractmethod
    def create_cache(self, page_size: int, head_dim: int) -> CacheShapes:
        ...

    # ------------------------------------------------------------------ runtime helpers
    def get_cache_meta_info(self, page_size: int, head_dim: int) -> CacheShapes:
        """The flow's own caches plus the mandatory ``"k"`` and ``"v"`` page blocks."""
        shapes = self.create_cache(page_size, head_dim)
        assert "k" not in shapes.keys()
        assert "v" not in shapes.keys()
        shapes["k"] = (page_size, head_dim)
        shapes["v"] = (page_size, head_dim)
        return shapes

    def get_token_ratio(self, page_size: int, head_dim: int) -> float:
        """Cache footprint relative to one K (or V) page block; K and V alone give 2.0."""
        unit = page_size * head_dim
        return sum((r * c) / unit for (r, c) in self.get_cache_meta_info(page_size, head_dim).values())

    def run_indexer_virtual(self, group_size: int, page_size: int, head_dim: int, device="cuda"):
        """Profile-pass the indexer on empty tensors and return its flop count per page.

        A fresh indexer context in profile mode is used, so no kernel runs; operators only
        validate shapes and add to the context's counters (``flow/flow.py:420-460``).
        """
        from ..abs import FORMAT, as_vtensor
        from ..indexer import Context as IndexerContext

        ctx = IndexerContext()
        ctx.group_size = group_size
        ctx.num_kv_heads = 1
        ctx.num_qo_heads = group_size
        ctx.head_dim = head_dim
        ctx.page_size = page_size
        ctx.max_num_pages = 0
        ctx.max_num_pages_per_request = 0
        dt = torch.bfloat16
        with torch.no_grad():
            q = as_vtensor(torch.empty((1, group_size, head_dim), device=device, dtype=dt), FORMAT.BATCHED)
            o = as_vtensor(torch.empty((0, 1, 1), device=device, dtype=dt), FORMAT.RAGGED)
            cache = {
                name: as_vtensor(torch.zeros((0, r, c), device=device, dtype=dt), FORMAT.PAGED)
                for name, (r, c) in self.get_cache_meta_info(page_size, head_dim).items()
            }
            self.forward_indexer(q, o, cache, ctx=ctx)
        return ctx._aux_total_flops
