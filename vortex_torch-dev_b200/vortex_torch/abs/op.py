"""Two-phase operator base class.

An operator instance is called as ``op(*args, ctx=ctx)``.  While the context is in profile
mode the call validates its (format-tagged) arguments, picks an implementation and allocates
the operator's persistent buffers; in execute mode it launches kernels on those buffers.
Contract of the reference's ``abs/op.py:8-108``.
"""
from __future__ import annotations

from abc import ABC, abstractmethod
from typing import Any

from ..utils import Mode
from .context_base import ContextBase


class vOp(ABC):
    def __init__(self) -> None:
        super().__init__()

    @abstractmethod
    def profile(self, *args: Any, ctx: ContextBase = None, **kwargs: Any) -> Any:
        raise NotImplementedError

    @abstractmethod
    def execute(self, *args: Any, ctx: ContextBase = None, **kwargs: Any) -> Any:
        raise NotImplementedError

    def __call__(self, *args: Any, ctx: ContextBase = None, **kwargs: Any) -> Any:
        mode = ctx.mode
        if mode is None or mode == Mode.execute:
            return self.execute(*args, ctx=ctx, **kwargs)
        if mode == Mode.profile:
            return self.profile(*args, ctx=ctx, **kwargs)
        raise ValueError(f"Unknown mode: {mode!r}, expected 'profile' or 'execute'")

    def _prefix(self) -> str:
        return f"{type(self).__name__}: "
