"""Bookkeeping for operator chains that can run as one fused kernel.

The indexer operators of the ``gqa_block_sparse_attention`` flow (``GeMM -> Softmax -> Max -> topK``) and of
the ``gqa_quest_sparse_attention`` flow (``Multiply x2 -> Maximum -> Sum -> Max -> topK``) each have a
stand-alone sm_100a kernel, and each chain as a whole has a fused one.  In the profile pass every operator
records itself on the tensor it returns; the final ``topK`` recognises a chain and claims its links
(``_fused_into``).  A claimed link does no work of its own in execute mode as long as the chain is intact:
every link's output has exactly one consumer (the next link) and nothing else read it.  Otherwise every link
runs its stand-alone kernel and ``topK`` selects from the scores it is handed - same bits either way.
"""
from __future__ import annotations

from typing import List, Optional, Tuple


def chain_of(t) -> List[Tuple[str, object]]:
    return list(getattr(t, "_vtx_chain", []))


def tag(t, chain: List[Tuple[str, object]], producer) -> None:
    t._vtx_chain = chain
    t._vtx_producer = producer  # lets vTensor notice plain torch reads of this intermediate


def note_consumer(t) -> None:
    """An operator that may be the next link of a chain consumes tensor ``t``."""
    prod = getattr(t, "_vtx_producer", None)
    if prod is not None and hasattr(prod, "_consumers"):
        prod._consumers += 1


def mark_read(t) -> None:
    """An operator that is never part of a fused chain reads tensor ``t``: its producer must really write it."""
    prod = getattr(t, "_vtx_producer", None)
    if prod is not None and hasattr(prod, "_score_read_elsewhere"):
        prod._score_read_elsewhere = True


class ChainedOp:
    """Mixin: state shared by operators that can run as a link of a fused chain."""

    _fused_into: Optional[object] = None  # the topK that claimed this link
    _score_read_elsewhere: bool = False
    _consumers: int = 0

    def _link_intact(self) -> bool:
        return not self._score_read_elsewhere and self._consumers <= 1

    def _runs_fused(self) -> bool:
        owner = self._fused_into
        return owner is not None and owner.chain_intact()
