"""Indexer-side operators: score pages against the query and pick the sparse page set.

Export list of the reference's ``indexer/__init__.py:49-71``; every name has an sm_100a kernel behind it.
The shipped flows' chains (``q.mean -> GeMV -> topK``, ``GeMM -> Softmax -> Max -> topK``,
``Multiply x2 -> Maximum -> Sum -> Max -> topK``) run as one fused kernel each; any other composition runs the
operators' stand-alone kernels.
"""
from .context import Context, get_ctx
from .elementwise import Abs, Add_Mul, Relu, Sigmoid, Silu
from .elementwise_binary import Add, Maximum, Minimum, Multiply
from .matmul import GeMM, GeMV
from .output_func import topK
from .reduce import L2Norm, Max, Mean, Min, Sum
from .save_load import Load, Save
from .scan import Normalize, Softmax
from .transpose import Transpose
from . import utils_sglang

__all__ = [
    "GeMM", "GeMV", "topK", "Max", "Mean", "Min", "L2Norm", "Sum", "Softmax", "Normalize", "Transpose",
    "Maximum", "Minimum", "Multiply", "Add", "Relu", "Sigmoid", "Silu", "Add_Mul", "Abs", "Save", "Load",
    "utils_sglang", "Context", "get_ctx",
]
