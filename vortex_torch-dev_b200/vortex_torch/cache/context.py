"""Cache context: page geometry of the KV pool, read by the cache-side operators
(reference: ``cache/context.py:7-60``)."""
from __future__ import annotations

from typing import Any

from ..abs import ContextBase


class Context(ContextBase):
    __slots__ = ContextBase.__slots__ + (
        "max_new_tokens_per_batch", "page_size", "total_num_pages", "head_dim", "head_num",
        "_aux_total_bytes", "_aux_total_flops",
    )

    def __init__(self) -> None:
        self._reset_slots("Cache")

    def create(self, parent: Any, model_runner: Any, *, overwrite: bool = False) -> "Context":
        """``parent`` is the KV pool (page_size, num_pages, head_num, head_dim)."""
        if self._created and not overwrite:
            raise RuntimeError("Context.create() already called; pass overwrite=True to reinitialize.")
        self.page_size = parent.page_size
        self.total_num_pages = parent.num_pages
        self.max_new_tokens_per_batch = max(model_runner.server_args.max_prefill_tokens,
                                            model_runner.req_to_token_pool.size)
        self.head_num = parent.head_num
        self.head_dim = parent.head_dim
        self._created = True
        return self
