"""``build_vflow``: instantiate a registered flow, optionally importing a user file first so
that its ``@register`` decorators run (reference: ``flow/loader.py:19-94``)."""
from __future__ import annotations

import importlib.util
import inspect
import os
import uuid
from types import ModuleType
from typing import Any, Dict, Optional

from .flow import vFlow
from .registry import RegistryError, get as _lookup, list_keys


class FlowLoadError(Exception):
    """The user file could not be imported, or the requested name is not registered."""


class FlowInitError(Exception):
    """Constructor arguments do not fit, or the constructor raised."""


def _load_module_from_file(file_path: str) -> ModuleType:
    """Execute ``file_path`` as a module under a one-off name (no caching, no name clashes)."""
    if not os.path.isfile(file_path):
        raise FlowLoadError(f"File does not exist: {file_path}")
    spec = importlib.util.spec_from_file_location(f"user_flow_{uuid.uuid4().hex}", file_path)
    if spec is None or spec.loader is None:
        raise FlowLoadError(f"Failed to create import spec for: {file_path}")
    module = importlib.util.module_from_spec(spec)
    try:
        spec.loader.exec_module(module)
    except Exception as exc:
        raise FlowLoadError(f"Failed to import user module: {exc}") from exc
    return module


def _validate_kwargs(cls: type, init_kwargs: Dict[str, Any]) -> None:
    """Bind the kwargs against ``cls.__init__`` so a mismatch is reported before construction."""
    try:
        inspect.signature(cls.__init__).bind_partial(None, **(init_kwargs or {}))
    except TypeError as exc:
        raise FlowInitError(f"Constructor arguments mismatch: {exc}") from exc


def build_vflow(selected: str, init_kwargs: Optional[Dict[str, Any]] = None,
                user_file: Optional[str] = None) -> vFlow:
    if user_file:
        _load_module_from_file(user_file)
    try:
        flow_cls = _lookup(selected)
    except RegistryError as exc:
        raise FlowLoadError(f"{exc} (available: {list_keys()})")
    kwargs = init_kwargs or {}
    _validate_kwargs(flow_cls, kwargs)
    try:
        return flow_cls(**kwargs)
    except Exception as exc:
        raise FlowInitError(f"Failed to instantiate: {exc}") from exc
