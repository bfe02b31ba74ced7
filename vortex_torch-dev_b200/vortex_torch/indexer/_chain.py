"""Bookkeeping for operator chains that only exist as one fused kernel.

The operators of the ``gqa_block_sparse_attention`` indexer (``GeMM -> Softmax -> Max -> topK``) have no
stand-alone sm_100a kernels: each records itself on the tensor it returns during the profile pass, the
final ``topK`` recognises the chain and owns the single fused launch.  An operator that is executed
outside a recognised chain fails loudly.
"""
from __future__ import annotations

from typing import List, Optional, Tuple


def chain_of(t) -> List[Tuple[str, object]]:
    return list(getattr(t, "_vtx_chain", []))


def tag(t, chain: List[Tuple[str, object]], producer) -> None:
    t._vtx_chain = chain
    t._vtx_producer = producer  # lets vTensor notice plain torch reads of this intermediate


class ChainedOp:
    """Mixin: state shared by operators that run only inside a fused chain."""

    _fused_into: Optional[object] = None
    _score_read_elsewhere: bool = False

    def _require_fused(self, what: str) -> None:
        if self._fused_into is None or self._score_read_elsewhere:
            raise NotImplementedError(
                f"vortex_torch.indexer.{what}: no stand-alone sm_100a kernel; it runs only as part of the chain "
                f"GeMM -> Softmax(dim=0) -> Max(dim=2) -> topK whose intermediates nothing else reads")
