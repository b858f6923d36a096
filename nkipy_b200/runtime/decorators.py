"""``@baremetal_jit``: trace, compile and run on the device at every call
(nkipy/src/nkipy/runtime/decorators.py:10-66 in the reference)."""

from __future__ import annotations

import functools

from ..core.compile import CompilationTarget, trace
from .execute import baremetal_run_traced_kernel


def baremetal_jit(func=None, *, backend: str = "hlo", additional_compiler_args: str = "",
                  target: CompilationTarget = CompilationTarget.DEFAULT):
    def wrap(fn):
        kernel = trace(fn, backend=backend)

        @functools.wraps(fn)
        def wrapper(*args, **kwargs):
            return baremetal_run_traced_kernel(kernel, *args, additional_compiler_args=additional_compiler_args,
                                               target=target, **kwargs)

        wrapper.kernel = kernel
        return wrapper

    return wrap(func) if func is not None else wrap
