"""Core abstractions: contexts, two-phase operators and format-tagged tensors."""
from .context_base import ContextBase
from .op import vOp
from .tensor import FORMAT, as_vtensor, vTensor

__all__ = ["ContextBase", "vOp", "vTensor", "as_vtensor", "FORMAT"]
