"""Operation dispatcher: one `Op` per frontend operation, implementations per backend.

Same contract as the reference (nkipy/src/nkipy/core/ops/_registry.py:12-99): calling
an `Op` picks the implementation registered for the active backend (`get_backend()`),
falls back to a backend-agnostic *composed* implementation built from other ops, and
raises `NotImplementedError` otherwise.  A "b200" / "nkigen" trace context reuses the
IR implementations registered under "hlo".
"""

from __future__ import annotations

from typing import Callable, Dict, Optional

from ..backend import get_backend

_ALIASES = {"b200": "hlo", "nkigen": "hlo"}


class Op:
    def __init__(self, name: str):
        self.name = name
        self._impls: Dict[str, Callable] = {}
        self._composed: Optional[Callable] = None

    def impl(self, backend: str) -> Callable:
        def decorator(fn: Callable) -> Callable:
            self._impls[backend] = fn
            return fn

        return decorator

    @property
    def composed_impl(self):
        def decorator(fn: Callable) -> Callable:
            self._composed = fn
            return fn

        return decorator

    def has_impl(self, backend: str) -> bool:
        return backend in self._impls or _ALIASES.get(backend) in self._impls or self._composed is not None

    def __call__(self, *args, **kwargs):
        backend = get_backend()
        fn = self._impls.get(backend)
        if fn is None:
            fn = self._impls.get(_ALIASES.get(backend, ""))
        if fn is None:
            fn = self._composed
        if fn is None:
            raise NotImplementedError(f"Operation '{self.name}' is not implemented for backend '{backend}'")
        out = fn(*args, **kwargs)
        if out is NotImplemented and fn is not self._composed and self._composed is not None:
            # a backend implementation may decline a case (an axis, a dtype): the composition covers it
            out = self._composed(*args, **kwargs)
        return out

    def __repr__(self) -> str:
        return f"<Op '{self.name}' backends={sorted(self._impls)}{' +composed' if self._composed else ''}>"
