"""Indexer context: the per-step page lists and the static sizes every indexer operator reads.

Field names and the ``create(parent, model_runner)`` contract are those of the reference's
``indexer/context.py:8-170``.  ``parent`` is the attention backend (it owns the index buffers);
``model_runner.server_args`` carries the ``vortex_*`` flags.
"""
from __future__ import annotations

from typing import Any, Final

import torch

from ..abs import ContextBase


class Context(ContextBase):
    __slots__ = ContextBase.__slots__ + (
        # page lists (int32 device tensors) and the active batch size
        "dense_kv_indices", "sparse_kv_indices", "dense_kv_indptr", "sparse_kv_indptr", "kv_last_page_len",
        "batch_size",
        # workload list for chunk-scheduled operators
        "winfo_q_indices", "winfo_kv_offsets", "winfo_kv_lens", "winfo_num_workloads", "winfo_chunk_size",
        "max_num_workloads", "max_chunk_size", "min_chunk_size",
        # attention shape
        "group_size", "num_kv_heads", "num_qo_heads", "head_dim",
        # device / paging
        "num_sms", "page_size", "max_num_pages", "max_num_pages_per_request",
        # selection parameters
        "indexer_dtype", "topk_val", "page_reserved_bos", "page_reserved_eos",
        # profile-pass counters
        "_aux_total_bytes", "_aux_total_flops",
        # a fused page selection that the runtime may fold into its attention launch (see defer_indexer)
        "_defer_indexer", "_pending_indexer",
    )

    def __init__(self) -> None:
        self._reset_slots("Indexer", {"batch_size": 0, "_defer_indexer": False, "_pending_indexer": None})

    # ---- deferred page selection (fusion of the indexer with the attention that follows it) ----
    def defer_indexer(self, enable: bool) -> None:
        """When enabled, a fused ``q.mean -> GeMV -> topK`` (or ``GeMM -> Softmax -> Max -> topK``) chain is
        recorded instead of launched, so that
        the caller's attention step can run selection and attention as one kernel.  The caller must call
        ``take_pending_indexer`` or ``flush_indexer`` before anything reads the sparse page list."""
        self.flush_indexer()
        self._defer_indexer = bool(enable)

    def take_pending_indexer(self):
        pend, self._pending_indexer = self._pending_indexer, None
        return pend

    def record_or_launch(self, selection) -> None:
        """Called by the operator that owns a fused page selection (`_deferred.PendingSelection`): keep it for the
        caller's attention step when that was asked for, else launch it now."""
        from .. import _deferred

        self.flush_indexer()
        if self._defer_indexer:
            self._pending_indexer = selection
            return
        _deferred.flush_all()
        selection.launch(self)

    def flush_indexer(self) -> None:
        pend = self.take_pending_indexer()
        if pend is not None:
            from .. import _deferred

            _deferred.flush_all()
            pend.launch(self)

    def run_sparse_layer(self, q, k_cache, v_cache, out, kv_last_page_len, sm_scale: float, cache_ctx=None,
                         workspace=None, early_prologue: bool = False) -> bool:
        """The attention step of a sparse layer, for a backend that called ``defer_indexer(True)`` before
        ``flow.forward_indexer`` (and ``cache_ctx.defer_append(True)`` before ``flow.forward_cache``).

        If the flow recorded a page selection on ``q`` that the one-launch layer kernel supports, this runs
        token write (when ``cache_ctx`` holds a matching recorded append) + selection + attention over the
        selected pages into ``out`` as ONE kernel and returns True.  Otherwise everything recorded is launched
        as the separate kernels, the sparse page list is complete on return, and the result is False: the
        caller then runs its own paged attention over ``sparse_kv_indptr / sparse_kv_indices``.
        Call order of the reference's hook: ``flow/algorithms.py:114-205`` (forward_cache, forward_indexer,
        then the backend's paged decode)."""
        from .. import _deferred

        sel = self.take_pending_indexer()
        if sel is None or not (_deferred._same(sel.q, q) and sel.out.data_ptr() == self.sparse_kv_indices.data_ptr()
                               and _deferred.sparse_layer_supported(sel, self, k_cache)):
            if sel is not None:
                self._pending_indexer = sel
                self.flush_indexer()
            if cache_ctx is not None:
                cache_ctx.flush_append()
            return False
        app = cache_ctx.take_pending_append() if cache_ctx is not None else None
        if app is not None and not _deferred.append_joins(app, sel, self, k_cache, v_cache, self.page_size):
            app.launch(cache_ctx)
            app = None
        _deferred.sparse_layer_launch(sel, app, self, k_cache, v_cache, out, kv_last_page_len, self.page_size, sm_scale,
                                      workspace=workspace, early_prologue=early_prologue)
        return True

    def set_batch_size(self, n: int) -> None:
        self.batch_size = n

    def create(self, parent: Any, model_runner: Any, *, overwrite: bool = False) -> "Context":
        """Fill the context once (single caller thread; pass ``overwrite=True`` to redo it)."""
        if self._created and not overwrite:
            raise RuntimeError("Context.create() already called; pass overwrite=True to reinitialize.")
        sa = model_runner.server_args
        P = sa.page_size
        longest = model_runner.model_config.context_len if sa.vortex_max_seq_lens < 0 else sa.vortex_max_seq_lens
        pages_per_req = (longest + P - 1) // P
        max_bs = int(model_runner.req_to_token_pool.size)

        self.dense_kv_indices, self.sparse_kv_indices = parent.kv_indices_decode[0], parent.kv_indices_decode[1]
        self.dense_kv_indptr, self.sparse_kv_indptr = parent.kv_indptr_decode[0], parent.kv_indptr_decode[1]
        self.kv_last_page_len = parent.kv_last_page_len_decode

        self.max_chunk_size = sa.vortex_lb_max_chunk_size
        self.min_chunk_size = sa.vortex_lb_min_chunk_size
        self.group_size = parent.group_size
        self.num_kv_heads = parent.num_kv_heads
        self.num_qo_heads = parent.num_qo_heads
        self.head_dim = parent.head_dim

        device = getattr(model_runner, "device", "cpu")
        dev = torch.device(device)
        self.num_sms = (torch.cuda.get_device_properties(dev).multi_processor_count
                        if dev.type == "cuda" and torch.cuda.is_available() else 0)
        self.page_size = P
        self.max_num_pages_per_request = pages_per_req
        self.max_num_pages = pages_per_req * max_bs * self.num_kv_heads

        self.topk_val = sa.vortex_topk_val
        dt = getattr(sa, "vortex_indexer_dtype", "float32")
        self.indexer_dtype = getattr(torch, dt, torch.float32) if isinstance(dt, str) else dt
        self.page_reserved_bos = sa.vortex_page_reserved_bos
        self.page_reserved_eos = sa.vortex_page_reserved_eos

        self.max_num_workloads = self.max_num_pages // max(1, sa.vortex_lb_min_chunk_size) + max_bs * self.num_kv_heads
        for slot in ("winfo_q_indices", "winfo_kv_offsets", "winfo_kv_lens"):
            setattr(self, slot, torch.zeros((self.max_num_workloads,), dtype=torch.int32, device=device))
        self.winfo_num_workloads = torch.zeros((1,), dtype=torch.int32, device=device)
        self.winfo_chunk_size = torch.zeros((1,), dtype=torch.int32, device=device)
        self._created = True
        return self


# Process-wide instance used by the serving hook (one attention backend per process).
ctx: Final[Context] = Context()


def get_ctx() -> Context:
    return ctx


__all__ = ["Context", "ctx", "get_ctx"]
