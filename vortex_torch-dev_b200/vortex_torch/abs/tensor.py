"""Format-tagged tensors.

``vTensor`` is a ``torch.Tensor`` subclass that carries a layout tag (``FORMAT``) through torch
operations: results inherit the tag, tags must agree, and a tagged tensor may not be combined
with an untagged one (python scalars are fine).  Behaviour of the reference's
``abs/tensor.py:8-165``.

Two private extras support kernel fusion in the indexer and change no visible result:

* the result of ``q.mean(dim=1, keepdim=True)`` on a BATCHED tensor is marked as a grouped-query
  mean, so that a following ``GeMV -> topK`` chain can be run as one fused kernel;
* when the runtime marks ``q`` with ``_vtx_allow_lazy_mean`` that mean is not launched at all:
  a view stands in for it and remembers ``q``; the fused kernel takes the mean itself, and any
  other torch operation that receives the stand-in first replaces it by the real mean.
"""
from __future__ import annotations

from enum import Enum
from typing import Any, Callable, Iterator, Optional

import torch


class FORMAT(Enum):
    BATCHED = 0  # [B, r, c]: one block per request/segment
    RAGGED = 1   # [S_packed, r, c]: per-page blocks packed segment after segment
    PAGED = 2    # [num_pages * H, r, c]: blocks addressed by physical cache row


def _tensors_in(obj: Any) -> Iterator[torch.Tensor]:
    if isinstance(obj, torch.Tensor):
        yield obj
    elif isinstance(obj, (list, tuple)):
        for item in obj:
            yield from _tensors_in(item)
    elif isinstance(obj, dict):
        for item in obj.values():
            yield from _tensors_in(item)


def _map_tensors(obj: Any, fn: Callable[[torch.Tensor], Any]) -> Any:
    if isinstance(obj, torch.Tensor):
        return fn(obj)
    if isinstance(obj, (list, tuple)):
        return type(obj)(_map_tensors(x, fn) for x in obj)
    if isinstance(obj, dict):
        return {k: _map_tensors(v, fn) for k, v in obj.items()}
    return obj


def _retag(result: Any, fmt: Optional["FORMAT"]) -> Any:
    if fmt is None:
        return result
    if isinstance(result, vTensor):
        result._format = fmt
        return result
    if isinstance(result, torch.Tensor):
        return vTensor._wrap(result, fmt)
    if isinstance(result, (list, tuple)):
        return type(result)(_retag(x, fmt) for x in result)
    if isinstance(result, dict):
        return {k: _retag(v, fmt) for k, v in result.items()}
    return result


def _metadata_functions():
    """Tensor accessors that look at shape/placement only and never at the data."""
    T = torch.Tensor
    fns = {T.dim, T.size, T.stride, T.numel, T.nelement, T.ndimension, T.is_contiguous, T.data_ptr,
           T.element_size, T.storage_offset, T.is_floating_point, T.is_complex, T.get_device}
    for prop in ("shape", "device", "dtype", "ndim", "is_cuda", "is_cpu", "requires_grad", "layout", "is_sparse",
                 "is_quantized", "is_meta", "names", "itemsize", "nbytes"):
        getter = getattr(getattr(T, prop, None), "__get__", None)
        if getter is not None:
            fns.add(getter)
    return fns


_METADATA_FUNCS = _metadata_functions()


def _is_group_mean_call(func, args, kwargs) -> bool:
    if func not in (torch.Tensor.mean, torch.mean) or not args:
        return False
    src = args[0]
    if not isinstance(src, vTensor) or src.dim() != 3 or src._format != FORMAT.BATCHED:
        return False
    rest = list(args[1:])
    dim = kwargs.get("dim", rest[0] if rest else None)
    keepdim = kwargs.get("keepdim", rest[1] if len(rest) > 1 else False)
    if isinstance(dim, (list, tuple)) and len(dim) == 1:
        dim = dim[0]
    return dim == 1 and keepdim is True and kwargs.get("dtype") is None and "out" not in kwargs


def _plain(t: torch.Tensor) -> torch.Tensor:
    """The same storage as an untagged ``torch.Tensor`` (no dispatch through ``__torch_function__``)."""
    with torch._C.DisableTorchFunctionSubclass():
        return t.as_subclass(torch.Tensor)


def lazy_group_mean_source(x: Any) -> Optional[torch.Tensor]:
    """The tensor ``q`` that ``x`` is the not-yet-computed grouped-query mean of, or None."""
    return getattr(x, "_vtx_lazy_src", None)


def canonical_group_mean(src: torch.Tensor) -> torch.Tensor:
    """``src.mean(dim=1, keepdim=True)`` of a 3-D tensor in the arithmetic every kernel of the library uses for
    the grouped-query mean: an fp32 sum over the group in ascending order from +0.0, one division by the group
    size, one rounding to the dtype.  (torch's own ``mean`` leaves the order of the sum to its reduction
    kernel; with a fixed order the un-fused path selects exactly the pages the fused kernels select.)"""
    acc = torch.zeros((src.shape[0], src.shape[2]), dtype=torch.float32, device=src.device)
    for g in range(src.shape[1]):
        acc = acc + src[:, g].to(torch.float32)
    return (acc / float(src.shape[1])).to(src.dtype).unsqueeze(1)


def materialize(x: Any) -> Any:
    """Replace a stand-in for ``q.mean(dim=1, keepdim=True)`` by the computed mean."""
    src = lazy_group_mean_source(x)
    if src is None:
        return x
    plain = canonical_group_mean(_plain(src))
    return vTensor._wrap(plain, x._format) if isinstance(x, vTensor) else plain


class vTensor(torch.Tensor):
    _format: FORMAT

    def __new__(cls, data, _format: FORMAT = FORMAT.BATCHED, **kwargs):
        if not isinstance(data, torch.Tensor):
            data = torch.as_tensor(data, **kwargs)
        return cls._wrap(data, _format)

    @classmethod
    def _wrap(cls, base: torch.Tensor, fmt: FORMAT) -> "vTensor":
        out = torch.Tensor._make_subclass(cls, base, base.requires_grad)
        out._format = fmt
        return out

    def __repr__(self):  # noqa: D105
        if lazy_group_mean_source(self) is not None:
            return materialize(self).__repr__()
        body = super().__repr__().replace(type(self).__name__, "Tensor")
        return f"vTensor(format={self._format}, {body})"

    def __reduce_ex__(self, protocol):
        real = materialize(self)
        return (_rebuild_vtensor, (torch.Tensor(real), real._format, real.requires_grad))

    @classmethod
    def __torch_function__(cls, func, types, args=(), kwargs=None):
        kwargs = kwargs or {}
        if not any(issubclass(t, vTensor) for t in types):
            return super().__torch_function__(func, types, args, kwargs)
        if func in _METADATA_FUNCS:  # shape/device/dtype queries: no data is read, nothing to check or tag
            return super().__torch_function__(func, types, args, kwargs)
        tagged, plain, lazy = set(), False, False
        for t in _tensors_in((args, kwargs)):
            if isinstance(t, vTensor):
                tagged.add(t._format)
                lazy = lazy or lazy_group_mean_source(t) is not None
                producer = getattr(t, "_vtx_producer", None)
                if producer is not None:  # an operator's output is read by plain torch code
                    producer._score_read_elsewhere = True
            else:
                plain = True
        if tagged and plain:
            raise RuntimeError("vTensor cannot operate with plain torch.Tensor in the same op.")
        if len(tagged) > 1:
            raise RuntimeError(f"vTensor _format mismatch in op: {tagged}")
        fmt = next(iter(tagged)) if tagged else None
        if lazy:
            args, kwargs = _map_tensors(args, materialize), _map_tensors(kwargs, materialize)
        if _is_group_mean_call(func, args, kwargs):
            src = args[0]
            if getattr(src, "_vtx_allow_lazy_mean", False):
                out = cls._wrap(_plain(src).narrow(1, 0, 1), fmt)
                out._vtx_lazy_src = src
            elif src.dim() == 3 and src.dtype in (torch.bfloat16, torch.float32, torch.float16):
                out = cls._wrap(canonical_group_mean(_plain(src)), fmt)
            else:
                out = _retag(super().__torch_function__(func, types, args, kwargs), fmt)
            out._vtx_origin = "group_mean"
            return out
        return _retag(super().__torch_function__(func, types, args, kwargs), fmt)


def _rebuild_vtensor(t: torch.Tensor, fmt: FORMAT, requires_grad: bool) -> vTensor:
    out = vTensor._wrap(t, fmt)
    out.requires_grad_(requires_grad)
    return out


def as_vtensor(x: Any, _format: FORMAT = FORMAT.BATCHED) -> vTensor:
    """Tag ``x`` (no copy).  An existing vTensor is re-tagged in place and returned."""
    if isinstance(x, vTensor):
        x._format = _format
        return x
    if not isinstance(x, torch.Tensor):
        x = torch.as_tensor(x)
    return vTensor._wrap(x, _format)
