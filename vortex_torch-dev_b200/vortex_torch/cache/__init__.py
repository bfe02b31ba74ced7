"""Cache-side operators: maintain per-page summaries when new tokens complete a page.

Export list of the reference's ``cache/__init__.py:27-42``; every name has an sm_100a kernel behind it.
``Mean``, ``Max`` and ``Min`` on PAGED caches (the ``CMean``/``CMax``/``CMin`` of the shipped flows) are the tuned path that
the runtime folds into its KV write and attention launches; the other operators and layouts run generic
page-completion kernels.
"""
from .context import Context
from .elementwise import Abs, Add_Mul, Relu, Sigmoid, Silu
from .elementwise_binary import Add, Maximum, Minimum, Multiply
from .matmul import GeMM
from .reduce import L2Norm, Max, Mean, Min
from .set_kv import set_kv_buffer_launcher

__all__ = [
    "set_kv_buffer_launcher", "Mean", "Max", "Min", "L2Norm", "GeMM", "Relu", "Silu", "Sigmoid", "Abs",
    "Add_Mul", "Maximum", "Minimum", "Multiply", "Add", "Context",
]
