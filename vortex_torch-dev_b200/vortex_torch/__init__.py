"""vortex_torch — host-side operator/plugin API of the Vortex sparse-attention decode path,
backed by hand-written sm_100a CUDA kernels reached through a C-ABI shared library.

The import surface mirrors the reference package (``vortex_torch/__init__.py:2-16``):
``indexer``, ``cache``, ``flow``, ``abs`` and ``__version__``; ``runtime`` is the stand-in
for the serving engine's attention-backend hook.
"""
from . import abs as abs
from . import cache as cache
from . import flow as flow
from . import indexer as indexer
from .version import __version__

__all__ = ["indexer", "cache", "flow", "abs", "__version__"]
