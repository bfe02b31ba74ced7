"""One-GPU decode runtime that calls a vFlow the way the serving engine's attention backend does."""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence

import torch

from .. import _cabi
from ..abs import FORMAT, as_vtensor
from ..cache import Context as CacheContext, set_kv_buffer_launcher
from ..flow import build_vflow, vFlow
from ..indexer import Context as IndexerContext, utils_sglang


@dataclass
class ServerArgs:
    """The engine flags the contexts read (reference: ``indexer/context.py:108-150``, README engine kwargs)."""
    page_size: int = 16
    vortex_max_seq_lens: int = -1
    vortex_lb_max_chunk_size: int = 64
    vortex_lb_min_chunk_size: int = 16
    vortex_topk_val: int = 30
    vortex_indexer_dtype: str = "bfloat16"
    vortex_page_reserved_bos: int = 1
    vortex_page_reserved_eos: int = 1
    vortex_layers_skip: List[int] = field(default_factory=lambda: [0])
    vortex_module_name: str = "block_sparse_attention"
    vortex_module_path: Optional[str] = None
    enable_vortex_sparsity: bool = True
    max_prefill_tokens: int = 16384


@dataclass
class ModelConfig:
    context_len: int


class ReqToTokenPool:
    """``req_to_token[slot, i]`` = cache slot of token i of the request in pool row ``slot``."""

    def __init__(self, size: int, max_context_len: int, device):
        self.size = size
        self.req_to_token = torch.zeros((size, max_context_len), dtype=torch.int32, device=device)


class ModelRunnerStub:
    def __init__(self, server_args: ServerArgs, context_len: int, max_bs: int, device):
        self.server_args = server_args
        self.model_config = ModelConfig(context_len)
        self.device = device
        self.req_to_token_pool = ReqToTokenPool(max_bs, context_len, device)


class KVPool:
    """Paged caches of every layer: ``buffers[layer][name]`` is ``[num_pages*H, rows, cols]``."""

    def __init__(self, num_layers: int, num_pages: int, head_num: int, head_dim: int, page_size: int,
                 shapes: Dict[str, tuple], dtype, device):
        self.page_size, self.num_pages, self.head_num, self.head_dim = page_size, num_pages, head_num, head_dim
        self.buffers: List[Dict[str, torch.Tensor]] = [
            {name: torch.zeros((num_pages * head_num, r, c), dtype=dtype, device=device)
             for name, (r, c) in shapes.items()}
            for _ in range(num_layers)
        ]


class AttentionBackendStub:
    """Owner of the decode index buffers (``[0]`` dense, ``[1]`` sparse), as the contexts expect."""

    def __init__(self, num_qo_heads: int, num_kv_heads: int, head_dim: int, max_bs: int, pages_per_req: int,
                 budget: int, device):
        self.num_qo_heads, self.num_kv_heads, self.head_dim = num_qo_heads, num_kv_heads, head_dim
        self.group_size = num_qo_heads // num_kv_heads
        segs = max_bs * num_kv_heads
        i32 = dict(dtype=torch.int32, device=device)
        self.kv_indices_decode = [torch.zeros(segs * pages_per_req, **i32),
                                  torch.zeros(segs * min(budget, pages_per_req), **i32)]
        self.kv_indptr_decode = [torch.zeros(segs + 1, **i32), torch.zeros(segs + 1, **i32)]
        self.kv_last_page_len_decode = torch.zeros(segs, **i32)


class VortexDecodeRuntime:
    """Paged-KV decode over ``num_layers`` attention layers with a vFlow choosing the pages.

    Layers listed in ``server_args.vortex_layers_skip`` attend to every page (dense lists); all
    other layers attend to the pages the flow's indexer selected.
    """

    def __init__(self, num_layers: int, num_qo_heads: int, num_kv_heads: int, head_dim: int, num_pages: int,
                 max_bs: int, context_len: int, server_args: Optional[ServerArgs] = None,
                 dtype=torch.bfloat16, device="cuda", flow: Optional[vFlow] = None, sm_scale: Optional[float] = None):
        self.sa = server_args or ServerArgs()
        self.device = torch.device(device)
        self.dtype = dtype
        self.num_layers = num_layers
        self.H, self.Hq, self.D = num_kv_heads, num_qo_heads, head_dim
        self.G = num_qo_heads // num_kv_heads
        self.P = self.sa.page_size
        self.sm_scale = 1.0 / math.sqrt(head_dim) if sm_scale is None else sm_scale
        self.flow = flow or build_vflow(self.sa.vortex_module_name, None, self.sa.vortex_module_path)
        self.skip = set(self.sa.vortex_layers_skip) if self.sa.enable_vortex_sparsity else set(range(num_layers))
        self.fuse_attention = True  # run the flow's page selection and the attention as one kernel when possible
        self.pdl_mode = 0           # programmatic dependent launch: 0 off, 1 on, 2 on + early prologue
        self._launches_since_plan = 0

        self.model_runner = ModelRunnerStub(self.sa, context_len, max_bs, self.device)
        longest = context_len if self.sa.vortex_max_seq_lens < 0 else self.sa.vortex_max_seq_lens
        pages_per_req = (longest + self.P - 1) // self.P
        budget = self.sa.vortex_topk_val + self.sa.vortex_page_reserved_bos + self.sa.vortex_page_reserved_eos
        self.backend = AttentionBackendStub(num_qo_heads, num_kv_heads, head_dim, max_bs, pages_per_req, budget,
                                            self.device)
        self.pool = KVPool(num_layers, num_pages, num_kv_heads, head_dim, self.P,
                           self.flow.get_cache_meta_info(self.P, head_dim), dtype, self.device)
        # Batches that cannot fill the GPU with one CTA per segment get their page lists split (bf16 only).
        segs = max_bs * num_kv_heads
        self.num_splits = 1
        if dtype == torch.bfloat16 and head_dim in (64, 128) and self.G in (1, 2, 4, 8) and self.device.type == "cuda":
            self.num_splits = max(1, min(8, 592 // max(1, segs)))
        self.split_workspace = None
        if self.num_splits > 1:
            nbytes = _cabi.splitkv_workspace_bytes(segs, self.G, head_dim, self.num_splits)
            self.split_workspace = torch.empty(nbytes // 4, dtype=torch.float32, device=self.device)
        self.ictx = IndexerContext().create(self.backend, self.model_runner)
        self.cctx = CacheContext().create(self.pool, self.model_runner)
        # scratch that lets the one-launch layer spread a long segment's scan over several CTAs
        self.layer_workspace = None
        if self.device.type == "cuda":
            nbytes = _cabi.sparse_layer_workspace_bytes(segs, pages_per_req, self.sa.vortex_topk_val,
                                                        self.sa.vortex_page_reserved_bos,
                                                        self.sa.vortex_page_reserved_eos)
            if nbytes > 0:
                self.layer_workspace = torch.zeros(nbytes // 4, dtype=torch.int32, device=self.device)
        self._profile(max_bs)

    # ------------------------------------------------------------------ profile pass
    def _profile(self, max_bs: int) -> None:
        """Call the flow once with format-tagged tensors so operators validate and allocate."""
        self.ictx.profile()
        self.cctx.profile()
        cache0 = self.pool.buffers[0]
        tagged = {k: as_vtensor(v, FORMAT.PAGED) for k, v in cache0.items()}
        q = as_vtensor(torch.zeros((max_bs * self.H, self.G, self.D), dtype=self.dtype, device=self.device),
                       FORMAT.BATCHED)
        o = as_vtensor(self.backend.kv_indices_decode[1].view(-1, 1, 1), FORMAT.RAGGED)
        loc = torch.zeros((1,), dtype=torch.int64, device=self.device)
        with torch.no_grad():
            self.flow.forward_indexer(q, o, tagged, ctx=self.ictx)
            self.flow.forward_cache(tagged, loc, ctx=self.cctx)
        self.ictx.execute()
        self.cctx.execute()

    # ------------------------------------------------------------------ one decode step
    def plan(self, cached_seq_lens: torch.Tensor, req_indices: torch.Tensor) -> None:
        self._launches_since_plan = 0
        _cabi.set_programmatic_launch(min(self.pdl_mode, 1))
        utils_sglang.plan_decode(cached_seq_lens, self.model_runner.req_to_token_pool.req_to_token, req_indices,
                                 self.ictx)

    def attention(self, q: torch.Tensor, layer: int, out: torch.Tensor, sparse: bool) -> torch.Tensor:
        b = self.backend
        which = 1 if sparse else 0
        eff_bs = self.ictx.batch_size * self.H
        cache = self.pool.buffers[layer]
        if sparse:
            # the early prologue reads the planner's outputs: allowed once a launch that waits for its
            # predecessor before releasing its successor separates us from the planner
            early = self.pdl_mode == 2 and self._launches_since_plan >= 1
            if self.ictx.run_sparse_layer(q, cache["k"], cache["v"], out, b.kv_last_page_len_decode, self.sm_scale,
                                          cache_ctx=self.cctx, workspace=self.layer_workspace, early_prologue=early):
                self._launches_since_plan += 1
                return out
        else:
            self.ictx.flush_indexer()
            self.cctx.flush_append()
        if self.num_splits > 1:
            _cabi.decode_gqa_splitkv(q, cache["k"], cache["v"], out, b.kv_indptr_decode[which],
                                     b.kv_indices_decode[which], b.kv_last_page_len_decode, eff_bs, self.P,
                                     self.sm_scale, self.num_splits, self.split_workspace)
        else:
            _cabi.decode_gqa(q, cache["k"], cache["v"], out, b.kv_indptr_decode[which], b.kv_indices_decode[which],
                             b.kv_last_page_len_decode, eff_bs, self.P, self.sm_scale)
        self._launches_since_plan += 1
        return out

    def layer(self, layer: int, q: torch.Tensor, new_k: torch.Tensor, new_v: torch.Tensor, loc: torch.Tensor,
              out: torch.Tensor) -> torch.Tensor:
        """KV write, cache maintenance, page selection and attention of one layer.

        ``q`` ``[bs, H_q, D]``, ``new_k``/``new_v`` ``[bs, H_kv, D]``, ``loc`` ``[bs]`` int64, ``out`` like ``q``.
        """
        cache = self.pool.buffers[layer]
        # The KV write is handed to the cache context so that the flow's first cache operator can fold
        # it into its own kernel; whatever is left is launched right after forward_cache.
        self.cctx.defer_append(self.fuse_attention and layer not in self.skip)
        self.cctx.defer_kv_write(cache["k"], cache["v"], new_k, new_v, loc, self.P, single_token_pages=True)
        self.flow.forward_cache(cache, loc, ctx=self.cctx)
        self.cctx.flush_kv_write(keep_append=True)
        qv = q.view(-1, self.G, self.D)
        ov = out.view(-1, self.G, self.D)
        if layer in self.skip:
            return self.attention(qv, layer, ov, sparse=False)
        qt = as_vtensor(qv, FORMAT.BATCHED)
        qt._vtx_allow_lazy_mean = True
        self.ictx.defer_indexer(self.fuse_attention)
        try:
            self.flow.forward_indexer(qt, self.backend.kv_indices_decode[1].view(-1, 1, 1), cache, ctx=self.ictx)
            return self.attention(qv, layer, ov, sparse=True)
        finally:
            self.ictx.defer_indexer(False)
            self.cctx.defer_append(False)

    def step(self, cached_seq_lens: torch.Tensor, req_indices: torch.Tensor, q: Sequence[torch.Tensor],
             new_k: Sequence[torch.Tensor], new_v: Sequence[torch.Tensor], loc: torch.Tensor,
             out: Sequence[torch.Tensor]) -> None:
        """One decode step over all layers; per-layer inputs are indexable by layer."""
        self.plan(cached_seq_lens, req_indices)
        for l in range(self.num_layers):
            self.layer(l, q[l], new_k[l], new_v[l], loc, out[l])


class GraphedDecodeStep:
    """A whole decode step (all layers) captured once as a CUDA graph and replayed per step.

    Two ways to drive it:

    * ``replay()`` — inputs already sit in the static device buffers (``seq_lens``, ``req_indices``,
      ``loc``, ``q``, ``new_k``, ``new_v``); outputs land in ``out``.
    * ``run_from_host(...)`` — the engine-facing call: copies the step's inputs from pinned host
      buffers, replays, copies the attention outputs back to pinned host memory and waits.
    """

    def __init__(self, rt: VortexDecodeRuntime, batch_size: int):
        self.rt = rt
        dev, dt = rt.device, rt.dtype
        L, bs = rt.num_layers, batch_size
        self.seq_lens = torch.zeros(bs, dtype=torch.int32, device=dev)
        self.req_indices = torch.zeros(bs, dtype=torch.int64, device=dev)
        self.loc = torch.zeros(bs, dtype=torch.int64, device=dev)
        self.q = torch.zeros(L, bs, rt.Hq, rt.D, dtype=dt, device=dev)
        self.new_k = torch.zeros(L, bs, rt.H, rt.D, dtype=dt, device=dev)
        self.new_v = torch.zeros(L, bs, rt.H, rt.D, dtype=dt, device=dev)
        self.out = torch.zeros(L, bs, rt.Hq, rt.D, dtype=dt, device=dev)
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self._host = None

    def _eager(self) -> None:
        self.rt.step(self.seq_lens, self.req_indices, self.q, self.new_k, self.new_v, self.loc, self.out)

    def capture(self, programmatic_launch=0) -> None:
        """Capture the step.  ``programmatic_launch``: 0 plain graph edges, 1 kernels chained by
        programmatic dependent launch (each waits for its whole predecessor), 2 additionally lets the
        fused layer kernels run their read-only prologue ahead of that wait."""
        self.rt.pdl_mode = int(programmatic_launch)
        try:
            self._capture()
        finally:
            self.rt.pdl_mode = 0
            _cabi.set_programmatic_launch(0)

    def _capture(self) -> None:
        side = torch.cuda.Stream(self.rt.device)
        side.wait_stream(torch.cuda.current_stream(self.rt.device))
        with torch.cuda.stream(side):
            self._eager()  # loads every kernel and sets launch attributes outside the capture
        torch.cuda.current_stream(self.rt.device).wait_stream(side)
        torch.cuda.synchronize(self.rt.device)
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            self._eager()

    def replay(self) -> None:
        if self.graph is None:
            self._eager()
        else:
            self.graph.replay()

    # ---- host-buffer path
    def host_buffers(self):
        """Pinned host twins of the step inputs and outputs (allocated on first use)."""
        if self._host is None:
            pin = lambda t: torch.zeros(t.shape, dtype=t.dtype).pin_memory()
            self._host = {n: pin(getattr(self, n)) for n in
                          ("seq_lens", "req_indices", "loc", "q", "new_k", "new_v", "out")}
        return self._host

    @property
    def h2d_bytes(self) -> int:
        return sum(getattr(self, n).numel() * getattr(self, n).element_size()
                   for n in ("seq_lens", "req_indices", "loc", "q", "new_k", "new_v"))

    @property
    def d2h_bytes(self) -> int:
        return self.out.numel() * self.out.element_size()

    def capture_host_pipeline(self, programmatic_launch=0, layers_per_gate: int = 7, first_group: int = 1,
                              last_group: int = 1, layers_per_output: Optional[int] = None) -> None:
        """Capture the host-buffer step as one graph in which the copies overlap the kernels.

        Three branches inside the graph: an input branch copies the step's pinned host inputs layer by
        layer, the compute branch starts a group of ``layers_per_gate`` layers as soon as that group's inputs
        have landed, and an output branch copies layer l's attention output back while layer l+1 computes.
        ``run_from_host`` replays it.  The inputs arrive far ahead of the compute branch (a layer's inputs
        take a few microseconds of PCIe time, the layer tens), so the gates cost nothing in waiting; they are
        kept few because a kernel that waits for a copy node cannot be chained to its predecessor by
        programmatic dependent launch.  The first input group holds only ``first_group`` layers, so that compute
        starts after a fraction of the inputs has crossed PCIe (the rest arrives under it), and the last
        ``last_group`` layers' outputs go back as a copy of their own, so that little is left to copy once the
        last kernel has finished; in between, outputs go back every ``layers_per_output`` layers (default: the
        input group size).
        """
        h = self.host_buffers()
        dev = self.rt.device
        self._eager()
        torch.cuda.synchronize(dev)
        self.rt.pdl_mode = int(programmatic_launch)
        try:
            L = self.rt.num_layers
            gate = max(1, int(layers_per_gate))
            first = min(L, max(1, int(first_group)))
            in_starts = [0] + list(range(first, L, gate))
            last = min(L, max(1, int(last_group)))
            og = gate if layers_per_output is None else max(1, int(layers_per_output))
            out_ends = sorted(set(list(range(first + og, L - last + 1, og)) + [first, L - last, L]) - {0})
            self._capture_host_pipeline(h, dev, in_starts, out_ends)
        finally:
            self.rt.pdl_mode = 0
            _cabi.set_programmatic_launch(0)

    def _capture_host_pipeline(self, h, dev, in_starts, out_ends) -> None:
        """``in_starts``: first layer of every input group; ``out_ends``: layer counts after which the outputs
        computed since the previous such point are copied back."""
        s_in, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
        L = self.rt.num_layers
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            main = torch.cuda.current_stream(dev)
            s_in.wait_stream(main)
            s_out.wait_stream(main)
            ev_meta = torch.cuda.Event()
            ev_in = {}
            with torch.cuda.stream(s_in):
                for n in ("seq_lens", "req_indices", "loc"):
                    getattr(self, n).copy_(h[n], non_blocking=True)
                ev_meta.record(s_in)
                for l0, l1 in zip(in_starts, in_starts[1:] + [L]):
                    # one copy per input tensor and group: the per-layer buffers of a group are contiguous
                    self.q[l0:l1].copy_(h["q"][l0:l1], non_blocking=True)
                    self.new_k[l0:l1].copy_(h["new_k"][l0:l1], non_blocking=True)
                    self.new_v[l0:l1].copy_(h["new_v"][l0:l1], non_blocking=True)
                    ev_in[l0] = torch.cuda.Event()
                    ev_in[l0].record(s_in)
            main.wait_event(ev_meta)
            self.rt.plan(self.seq_lens, self.req_indices)
            for l in range(L):
                if l in ev_in:
                    main.wait_event(ev_in[l])
                self.rt.layer(l, self.q[l], self.new_k[l], self.new_v[l], self.loc, self.out[l])
                if l + 1 in out_ends:
                    # outputs go back group by group too, while the next group computes
                    l0 = max([e for e in out_ends if e <= l], default=0)
                    ev = torch.cuda.Event()
                    ev.record(main)
                    s_out.wait_event(ev)
                    with torch.cuda.stream(s_out):
                        h["out"][l0:l + 1].copy_(self.out[l0:l + 1], non_blocking=True)
            main.wait_stream(s_in)
            main.wait_stream(s_out)
        self.graph_host = g

    def run_from_host(self, wait: bool = True):
        h = self.host_buffers()
        if getattr(self, "graph_host", None) is not None:
            self.graph_host.replay()
            if wait:
                torch.cuda.current_stream(self.rt.device).synchronize()
            return h["out"]
        for n in ("seq_lens", "req_indices", "loc", "q", "new_k", "new_v"):
            getattr(self, n).copy_(h[n], non_blocking=True)
        self.replay()
        h["out"].copy_(self.out, non_blocking=True)
        if wait:
            torch.cuda.current_stream(self.rt.device).synchronize()
        return h["out"]
