"""Registry of deferred launches.

The runtime may ask a context to record a launch instead of issuing it, so that a later call can run it
as part of one fused kernel.  Every code path that launches eagerly and could observe the deferred
work's results calls ``flush_all()`` first, which issues whatever is still pending, in registration order.
"""
from __future__ import annotations

from typing import Callable, List

_flushers: List[Callable[[], None]] = []


def register(flush: Callable[[], None]) -> None:
    if flush not in _flushers:
        _flushers.append(flush)


def flush_all() -> None:
    for f in list(_flushers):
        f()
