"""Shared pieces of the cache-side operators: operand layouts and the internal RAGGED output buffer."""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from ..abs import FORMAT, as_vtensor, vTensor

_CACHE_FORMATS = (FORMAT.PAGED, FORMAT.RAGGED)


def check_operand(prefix: str, name: str, t) -> None:
    assert isinstance(t, vTensor), f"{prefix}{name} must be vTensor, got {type(t)}"
    assert t.dim() == 3, f"{prefix}{name} must be 3D, got ndim={t.dim()} shape={tuple(t.shape)}"
    assert t._format in _CACHE_FORMATS, (
        f"{prefix}no implementation for {name}._format={t._format}. Available: {list(_CACHE_FORMATS)}")
    if t.dtype != torch.bfloat16:
        raise NotImplementedError(f"{prefix}the cache-side kernels are built for bfloat16, got {t.dtype}")


def resolve_output(prefix: str, x: vTensor, output: Optional[vTensor], inner: Tuple[int, int], ctx):
    """The reference's policy (cache/reduce.py:172-297): a given ``output`` fixes the layout; without one the
    operator owns a RAGGED buffer with one block per (new token, head)."""
    if output is not None:
        check_operand(prefix, "output", output)
        assert tuple(output.shape[1:]) == tuple(inner), (
            f"{prefix}output shape mismatch. Expected (*,{inner[0]},{inner[1]}), got {tuple(output.shape)}")
        assert x.device == output.device, (
            f"{prefix}x and output must be on the same device (x.device={x.device}, output.device={output.device})")
        return output, None
    buf = torch.empty((ctx.max_new_tokens_per_batch * ctx.head_num, inner[0], inner[1]), device=x.device, dtype=x.dtype)
    ctx.add_aux_memory(buf)
    return as_vtensor(buf, FORMAT.RAGGED), buf
