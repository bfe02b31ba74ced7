"""Stand-in for the serving engine's attention-backend hook.

The reference is driven by a patched SGLang whose source is not part of its tree; this package
plays that role for tests, benchmarks and examples: it owns the paged KV pool and the per-step
index buffers, creates the two contexts from objects that expose exactly the attributes the
reference's ``Context.create`` methods read, runs the profile pass, and drives one decode step
(plan -> per layer: KV write, ``forward_cache``, ``forward_indexer``, paged decode attention).
"""
from .engine import (AttentionBackendStub, GraphedDecodeStep, KVPool, ModelConfig, ModelRunnerStub, ReqToTokenPool, ServerArgs,
                     VortexDecodeRuntime)
from .sharding import (Shard, balance_requests, choose_head_shards, gather_for_verification, head_range,
                       local_row_to_global, shard_grid, slice_heads)

__all__ = ["ServerArgs", "ModelConfig", "ReqToTokenPool", "ModelRunnerStub", "KVPool", "AttentionBackendStub",
           "VortexDecodeRuntime", "GraphedDecodeStep", "balance_requests", "gather_for_verification", "Shard", "shard_grid",
           "head_range", "choose_head_shards", "slice_heads", "local_row_to_global"]
