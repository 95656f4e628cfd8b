"""Backend registry: name -> backend object, with lazy loading of the built-in one.

The same idiom as the reference's ``pipeline/registry.py:18-41`` (there it keys frontend
adapters): ``register(obj)`` stores by ``obj.name``; ``get(name)`` imports the module that
registers a built-in backend on first use and raises ``KeyError`` for unknown names.
"""

from __future__ import annotations

import importlib
from typing import Any, Dict

_REGISTRY: Dict[str, Any] = {}
_LAZY = {"b200": "intent_ir_b200.backend"}


def register(backend: Any) -> None:
    _REGISTRY[backend.name] = backend


def get(name: str) -> Any:
    cause = None
    if name not in _REGISTRY and name in _LAZY:
        try:
            importlib.import_module(_LAZY[name])
        except Exception as e:  # the KeyError below is the uniform failure; it carries the reason
            cause = e
    if name not in _REGISTRY:
        if cause is not None:
            raise KeyError(f"backend not registered: {name} (importing {_LAZY[name]} failed: {type(cause).__name__}: {cause})") from cause
        raise KeyError(f"backend not registered: {name}")
    return _REGISTRY[name]


__all__ = ["register", "get"]
