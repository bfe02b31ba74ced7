"""Cache-side operators: maintain per-page summaries when new tokens complete a page.

Export list of the reference's ``cache/__init__.py:27-42``.  Built on sm_100a: ``Mean``, ``Max``, ``Min`` (the
``CMean``/``CMax``/``CMin`` of the shipped flows), ``Context`` and ``set_kv_buffer_launcher``; the other names are
placeholders that raise ``NotImplementedError`` when used.
"""
from ..indexer._unbuilt import unbuilt as _unbuilt
from .context import Context
from .reduce import Max, Mean, Min
from .set_kv import set_kv_buffer_launcher

_W = "cache"
L2Norm = _unbuilt("L2Norm", _W)
GeMM = _unbuilt("GeMM", _W)
Relu, Silu, Sigmoid, Abs, Add_Mul = (_unbuilt(n, _W) for n in ("Relu", "Silu", "Sigmoid", "Abs", "Add_Mul"))
Maximum, Minimum, Multiply, Add = (_unbuilt(n, _W) for n in ("Maximum", "Minimum", "Multiply", "Add"))

__all__ = [
    "set_kv_buffer_launcher", "Mean", "Max", "Min", "L2Norm", "GeMM", "Relu", "Silu", "Sigmoid", "Abs",
    "Add_Mul", "Maximum", "Minimum", "Multiply", "Add", "Context",
]
