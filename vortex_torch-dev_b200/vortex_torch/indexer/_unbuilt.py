"""Placeholders for indexer operators that are exported by name but have no sm_100a kernel yet.

They can be constructed (shipped flows build all their operators in ``__init__``) and fail with
``NotImplementedError`` the first time they are profiled or executed.
"""
from __future__ import annotations

from ..abs import vOp


def unbuilt(name: str, where: str):
    class _Unbuilt(vOp):
        def __init__(self, *args, **kwargs):
            super().__init__()
            self._ctor = (args, kwargs)

        def _fail(self):
            raise NotImplementedError(
                f"vortex_torch.{where}.{name} has no sm_100a kernel in this build; only the operators of the "
                f"block_sparse_attention flow (GeMV, topK, cache Mean) are built")

        def profile(self, *args, ctx=None, **kwargs):
            self._fail()

        def execute(self, *args, ctx=None, **kwargs):
            self._fail()

    _Unbuilt.__name__ = _Unbuilt.__qualname__ = name
    return _Unbuilt
