"""Three-stage execution of a kernel: NumPy (CPU direct mode) -> trace + compile (nvcc, works without a
GPU) -> device run + comparison (reference: tools/kernel_agent/executor.py:49-123)."""

from __future__ import annotations

import dataclasses
import traceback
from typing import Callable, Dict, Optional, Sequence

import numpy as np


@dataclasses.dataclass
class ExecutionResult:
    numpy_ok: bool = False
    compile_ok: bool = False
    hardware_ok: Optional[bool] = None          # None = no GPU available, stage skipped
    numerics_ok: Optional[bool] = None
    max_abs_err: Optional[float] = None
    error_stage: Optional[str] = None
    error: Optional[str] = None

    @property
    def passed(self) -> bool:
        return self.numpy_ok and self.compile_ok and self.hardware_ok in (True, None) and self.numerics_ok in (True, None)

    def as_dict(self) -> Dict:
        return dataclasses.asdict(self)


def gpu_available() -> bool:
    try:
        import torch

        return torch.cuda.is_available()
    except Exception:
        return False


def compare(got, want, rtol: float, atol: float):
    got = got if isinstance(got, (tuple, list)) else (got,)
    want = want if isinstance(want, (tuple, list)) else (want,)
    worst = 0.0
    ok = len(got) == len(want)
    for g, w in zip(got, want):
        g, w = np.asarray(g), np.asarray(w)
        if g.shape != w.shape:
            return False, float("inf")
        if g.size == 0:
            continue
        gf, wf = g.astype(np.float64), w.astype(np.float64)
        worst = max(worst, float(np.nanmax(np.abs(gf - wf))))
        ok = ok and bool(np.allclose(gf, wf, rtol=rtol, atol=atol, equal_nan=True))
    return ok, worst


def run_kernel(fn: Callable, inputs: Sequence[np.ndarray], rtol: float = 1e-3, atol: float = 1e-3,
               use_gpu: Optional[bool] = None) -> ExecutionResult:
    import copy

    res = ExecutionResult()
    try:
        want = fn(*copy.deepcopy(list(inputs)))
        res.numpy_ok = True
    except Exception:
        res.error_stage, res.error = "numpy", traceback.format_exc(limit=3)
        return res
    try:
        from nkipy_b200.compiler.codegen import lower_to_cuda
        from nkipy_b200.core.compile import trace

        traced = trace(fn)
        graph = traced.specialize(*inputs)
        lower_to_cuda(graph)
        res.compile_ok = True
    except Exception:
        res.error_stage, res.error = "compile", traceback.format_exc(limit=3)
        return res
    if use_gpu is None:
        use_gpu = gpu_available()
    if not use_gpu:
        # no device: the IR interpreter stands in for the device so that the traced graph is still checked
        try:
            from nkipy_b200.core.interp import evaluate as run_graph

            got = run_graph(graph, list(inputs))
            res.numerics_ok, res.max_abs_err = compare(got, want, rtol, atol)
            if not res.numerics_ok:
                res.error_stage, res.error = "interpreter", f"max abs err {res.max_abs_err}"
        except Exception:
            res.error_stage, res.error = "interpreter", traceback.format_exc(limit=3)
            res.numerics_ok = False
        return res
    try:
        from nkipy_b200.runtime import baremetal_run_traced_kernel

        got = baremetal_run_traced_kernel(fn, *copy.deepcopy(list(inputs)))
        res.hardware_ok = True
        res.numerics_ok, res.max_abs_err = compare(got, want, rtol, atol)
        if not res.numerics_ok:
            res.error_stage, res.error = "numerics", f"max abs err {res.max_abs_err}"
    except Exception:
        res.hardware_ok = False
        res.error_stage, res.error = "hardware", traceback.format_exc(limit=3)
    return res
