"""Cache context: page geometry of the KV pool, read by the cache-side operators
(reference: ``cache/context.py:7-60``)."""
from __future__ import annotations

from typing import Any

from ..abs import ContextBase


class Context(ContextBase):
    __slots__ = ContextBase.__slots__ + (
        "max_new_tokens_per_batch", "page_size", "total_num_pages", "head_dim", "head_num",
        "_aux_total_bytes", "_aux_total_flops",
        # a KV write handed over by the runtime that the first cache operator may fuse with its own kernel
        "_pending_kv",
        # a fused KV write + page mean that the runtime may fold into its attention launch (see defer_append)
        "_defer_append", "_pending_append",
    )

    def __init__(self) -> None:
        self._reset_slots("Cache", {"_pending_kv": None, "_defer_append": False, "_pending_append": None})

    # ---- deferred append (KV write + page mean folded into the layer's attention kernel) ----
    def defer_append(self, enable: bool) -> None:
        """When enabled, a KV write that a ``Mean(dim=1)`` over the same K cache absorbed is recorded
        instead of launched; the runtime's attention step takes it (``take_pending_append``) or it is
        issued by ``flush_append`` / ``_deferred.flush_all`` before anything could read its results."""
        from .. import _deferred

        self.flush_append()
        self._defer_append = bool(enable)
        if enable:
            _deferred.register(self.flush_append)

    def take_pending_append(self):
        pend, self._pending_append = self._pending_append, None
        return pend

    def flush_append(self) -> None:
        pend = self.take_pending_append()
        if pend is not None:
            pend.launch(self)

    # ---- deferred KV write (fusion of set_kv with the flow's first cache operator) ----
    def defer_kv_write(self, k_cache, v_cache, new_k, new_v, loc, page_size: int,
                       single_token_pages: bool = False, page_ordered: bool = False) -> None:
        """Record a KV write instead of launching it.  The next cache operator either folds it into
        its own kernel (``Mean(dim=1)`` over the same K cache and ``loc``) or launches it first;
        the caller must call ``flush_kv_write`` after ``forward_cache`` in case no operator ran.

        ``single_token_pages``: the caller guarantees that no two slots of ``loc`` fall into the same
        page (a decode step: one new token per request).  ``page_ordered``: the rows of one page that this
        write holds are consecutive entries of ``loc`` in ascending slot order (a prefill).  With either
        guarantee the write may be folded into the mean (one launch); only the first also allows folding
        both into the layer's attention launch.  Without a guarantee the write is launched on its own."""
        from .._deferred import PendingKVWrite

        self.flush_kv_write()
        mode = "single" if single_token_pages else ("ordered" if page_ordered else None)
        self._pending_kv = PendingKVWrite(k_cache, v_cache, new_k, new_v, loc, page_size, mode)

    def flush_kv_write(self, keep_append: bool = False) -> None:
        """Launch a recorded write that no operator took.  ``keep_append``: leave a recorded append (write +
        page summary) for the caller's attention step instead of launching it here."""
        if not keep_append:
            self.flush_append()
        pend, self._pending_kv = self._pending_kv, None
        if pend is not None:
            pend.launch()

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
