"""Small enums and sentinels shared by the operator packages.

Same names and values as the reference's ``vortex_torch/utils.py:3-31`` so user flow files
that import them keep working.
"""
from enum import Enum


class _Unset:
    """Type of the ``UNSET`` sentinel: a context slot that ``create`` has not filled yet."""

    _inst = None

    def __new__(cls):
        if cls._inst is None:
            cls._inst = super().__new__(cls)
        return cls._inst

    def __repr__(self) -> str:
        return "UNSET"

    def __bool__(self) -> bool:
        return False


UNSET = _Unset()


class Mode(Enum):
    profile = 0
    execute = 1


class ReduceType(Enum):
    Mean = 0
    Max = 1
    Min = 2
    L2Norm = 3
    Sum = 4


class ElementwiseBinaryOpType(Enum):
    Maximum = 0
    Minimum = 1
    Add = 2
    Mul = 3


class ElementwiseOpType(Enum):
    Relu = 0
    Sigmoid = 1
    Silu = 2
    Abs = 3
    Add_Mul = 4
