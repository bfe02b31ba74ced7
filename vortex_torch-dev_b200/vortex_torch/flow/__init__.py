"""Plugin API for sparse-attention algorithms: ``vFlow``, ``register``, ``build_vflow`` and the
shipped ``algorithms`` (reference surface: ``flow/__init__.py:33-42``)."""
from .flow import vFlow
from .registry import register
from .loader import build_vflow
from . import algorithms

__all__ = ["vFlow", "register", "build_vflow", "algorithms"]
