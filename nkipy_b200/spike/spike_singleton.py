"""Process-wide runtime instance.

`configure(visible_cores=...)` restricts which GPUs the process may use (it sets
``CUDA_VISIBLE_DEVICES`` and therefore must run before the runtime starts),
`get_spike_singleton()` creates the runtime on first use (thread-safe) and registers an
``atexit`` hook that closes it before interpreter teardown, `reset()` closes it and
invalidates every tensor / model created from it.  Mirrors
spike/src/spike/spike_singleton.py:27-163 of the reference.
"""

from __future__ import annotations

import atexit
import os
import threading
import warnings
from typing import Iterable, Optional

_lock = threading.Lock()
_instance = None
_device_ordinal = -1


def _native():
    """The C++ runtime module; rebuilt first when its sources (or the argument-block header it shares
    with the kernels) changed since the in-tree binary was made and a compiler is available."""
    import importlib
    import shutil

    if "nkipy_b200.spike._spike" not in __import__("sys").modules and shutil.which("g++"):
        try:
            from ..runtime.native import build

            build()            # no-op when the stamp matches
        except Exception:      # fall back to the binary that is there
            pass
    try:
        return importlib.import_module("nkipy_b200.spike._spike")
    except ImportError:
        from ..runtime.native import build

        build()
        return importlib.import_module("nkipy_b200.spike._spike")


def configure(visible_cores: Optional[Iterable[int]] = None, device_ordinal: Optional[int] = None) -> None:
    """Choose the devices before the runtime is created."""
    global _device_ordinal
    with _lock:
        if _instance is not None:
            raise RuntimeError("configure() must be called before the runtime is initialised; call reset() first")
        if visible_cores is not None:
            os.environ["CUDA_VISIBLE_DEVICES"] = ",".join(str(int(c)) for c in visible_cores)
        if device_ordinal is not None:
            _device_ordinal = int(device_ordinal)


def get_spike_singleton():
    global _instance
    if _instance is None:
        with _lock:
            if _instance is None:
                _instance = _native().Spike(0, _device_ordinal)
                atexit.register(_close_at_exit)
    return _instance


def is_initialised() -> bool:
    return _instance is not None


def _close_at_exit():
    global _instance
    if _instance is not None:
        try:
            _instance.close()
        finally:
            _instance = None


def reset() -> None:
    """Close the runtime.  Tensors and models created from it become invalid."""
    global _instance
    with _lock:
        if _instance is not None:
            warnings.warn("Resetting the device runtime invalidates all existing tensors and models", stacklevel=2)
            _instance.close()
            _instance = None


def visible_device_count() -> int:
    return _native().Spike.get_visible_neuron_core_count()
