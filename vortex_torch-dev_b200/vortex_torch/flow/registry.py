"""Name -> flow class registry filled by the ``@register("name")`` decorator
(reference: ``flow/registry.py:6-41``)."""
from __future__ import annotations

from typing import Dict, List, Type

from .flow import vFlow

_REGISTRY: Dict[str, Type[vFlow]] = {}


class RegistryError(Exception):
    """Bad registration (not a vFlow, duplicate name) or unknown name on lookup."""


def register(name: str):
    def _decorate(cls: Type[vFlow]) -> Type[vFlow]:
        if not (isinstance(cls, type) and issubclass(cls, vFlow)):
            raise RegistryError(f"{getattr(cls, '__name__', cls)} must inherit from vFlow")
        if name in _REGISTRY:
            raise RegistryError(f"Registration name '{name}' already exists")
        _REGISTRY[name] = cls
        return cls

    return _decorate


def get(name: str) -> Type[vFlow]:
    if name not in _REGISTRY:
        raise RegistryError(f"Registration name '{name}' not found")
    return _REGISTRY[name]


def has(name: str) -> bool:
    return name in _REGISTRY


def list_keys() -> List[str]:
    return list(_REGISTRY)
