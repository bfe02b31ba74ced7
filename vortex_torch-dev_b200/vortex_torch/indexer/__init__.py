"""Indexer-side operators: score pages against the query and pick the sparse page set.

Export list of the reference's ``indexer/__init__.py:49-71``.  Built on sm_100a: ``GeMV``,
``topK``, ``Context``/``get_ctx``, ``utils_sglang`` and - as links of one fused kernel - ``GeMM``,
``Softmax`` and ``Max(dim=2)``; the unary elementwise family (``Relu``, ``Sigmoid``, ``Silu``, ``Abs``,
``Add_Mul``) and, on two RAGGED tensors, ``Add`` and ``Minimum``; the other names are placeholders that raise ``NotImplementedError`` when used.
"""
from ._unbuilt import unbuilt as _unbuilt
from .context import Context, get_ctx
from .elementwise import Abs, Add_Mul, Relu, Sigmoid, Silu
from .elementwise_binary import Add, Maximum, Minimum, Multiply
from .matmul import GeMM, GeMV
from .output_func import topK
from .reduce import L2Norm, Max, Mean, Min, Sum
from .scan import Normalize, Softmax
from . import utils_sglang

_W = "indexer"
Transpose = _unbuilt("Transpose", _W)
Save, Load = _unbuilt("Save", _W), _unbuilt("Load", _W)

__all__ = [
    "GeMM", "GeMV", "topK", "Max", "Mean", "Min", "L2Norm", "Sum", "Softmax", "Normalize", "Transpose",
    "Maximum", "Minimum", "Multiply", "Add", "Relu", "Sigmoid", "Silu", "Add_Mul", "Abs", "Save", "Load",
    "utils_sglang", "Context", "get_ctx",
]
