"""Base class of the indexer and cache contexts.

Mirrors the contract of the reference's ``abs/context_base.py:7-185``: a slotted object with a
``mode`` switch (profile / execute), a ``created`` flag set by ``create`` and two running
counters that operators feed during the profile pass (auxiliary bytes and flops).
"""
from __future__ import annotations

from abc import ABC, abstractmethod
from typing import Any, List, Union

import torch

from ..utils import UNSET, Mode


class ContextBase(ABC):
    __slots__ = ("name", "mode", "_created")

    # Subclasses list extra slots; these defaults apply to every context.
    _SLOT_DEFAULTS = {"_created": False, "_aux_total_bytes": 0, "_aux_total_flops": 0, "mode": Mode.profile}

    def _reset_slots(self, name: str, extra_defaults: dict | None = None) -> None:
        defaults = dict(self._SLOT_DEFAULTS)
        defaults["name"] = name
        if extra_defaults:
            defaults.update(extra_defaults)
        for slot in self.__slots__:
            object.__setattr__(self, slot, defaults.get(slot, UNSET))

    @property
    def created(self) -> bool:
        return self._created

    @abstractmethod
    def create(self, *args: Any, **kwargs: Any) -> "ContextBase":
        """Fill the context from the serving runtime's objects; returns ``self``."""
        raise NotImplementedError

    # ---- mode switch (operators dispatch on it, see vOp.__call__) ----
    def profile(self) -> None:
        self.mode = Mode.profile

    def execute(self) -> None:
        self.mode = Mode.execute

    # ---- bookkeeping ----
    def assert_created(self) -> None:
        if not self._created:
            raise RuntimeError("Context is not created yet.")

    def missing(self) -> List[str]:
        return [s for s in self.__slots__ if s != "_created" and getattr(self, s) is UNSET]

    def add_aux_memory(self, obj: Union[int, torch.Tensor]) -> int:
        """Count a scratch buffer (tensor or byte count) allocated by an operator's profile pass."""
        if isinstance(obj, torch.Tensor):
            nbytes = obj.element_size() * obj.nelement()
        elif isinstance(obj, int) and not isinstance(obj, bool):
            nbytes = obj
        else:
            raise TypeError("add_aux_memory expects an int (bytes) or a torch.Tensor")
        if nbytes < 0:
            raise ValueError("nbytes must be non-negative")
        self._aux_total_bytes += int(nbytes)
        return int(nbytes)

    def add_aux_flops(self, nflops: int) -> None:
        self._aux_total_flops += nflops

    def clear_aux_memory(self) -> None:
        self._aux_total_bytes = 0

    def clear_aux_flops(self) -> None:
        self._aux_total_flops = 0

    def summary(self) -> None:
        """Kept for API parity; the reference's implementation returns before printing anything."""
        return None
