"""Context-manager executor for compiled kernels: `run(...)` and `benchmark(...)`
(nkipy/src/nkipy/runtime/baremetal_executor.py:19-197 in the reference)."""

from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Any, Dict, Optional

import numpy as np

from ..core.ir import Graph
from ..core.trace import NKIPyKernel
from ..spike.spike_model import BenchmarkResult
from .device_kernel import DeviceKernel
from .device_tensor import DeviceTensor


@dataclass
class CompiledKernel:
    traced_kernel: NKIPyKernel
    compiled_artifact: str          # path of the cubin

    @property
    def ir(self) -> Graph:
        return self.traced_kernel._code


class BaremetalExecutor:
    def __init__(self, verbose: int = 0):
        self.verbose = verbose
        self._loaded: Dict[str, DeviceKernel] = {}

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        for m in self._loaded.values():
            try:
                m.unload()
            except Exception:
                pass
        self._loaded.clear()
        return False

    def _model(self, ck: CompiledKernel) -> DeviceKernel:
        if ck.compiled_artifact not in self._loaded:
            self._loaded[ck.compiled_artifact] = DeviceKernel.load_from_neff(ck.compiled_artifact)
        return self._loaded[ck.compiled_artifact]

    def _tensors(self, ck: CompiledKernel, args):
        ir = ck.ir
        arrays = [a for a in args if isinstance(a, np.ndarray)]
        inputs = {p.name: DeviceTensor.from_numpy(np.ascontiguousarray(a.astype(p.dtype, copy=False)), p.name)
                  for p, a in zip(ir.inputs, arrays)}
        alias = {a.output_index: ir.inputs[a.param_index].name for a in ir.aliases}
        outputs = {}
        for i, o in enumerate(ir.outputs):
            outputs[o.name] = inputs[alias[i]] if i in alias else DeviceTensor.empty(o.shape, o.dtype, o.name)
        return inputs, outputs

    def run(self, ck: CompiledKernel, *args, save_trace: bool = False, artifacts_dir: Optional[str] = None):
        model = self._model(ck)
        inputs, outputs = self._tensors(ck, args)
        ntff = os.path.join(artifacts_dir, "profile.trace.json") if (save_trace and artifacts_dir) else None
        model(inputs, outputs, save_trace=save_trace, ntff_name=ntff)
        ir = ck.ir
        res = [outputs[o.name].numpy() for i, o in enumerate(ir.outputs) if i not in ir.auto_aliased_indices]
        return res[0] if len(res) == 1 else tuple(res)

    def benchmark(self, ck: CompiledKernel, *args, warmup_iterations: int = 5, benchmark_iterations: int = 100,
                  mode: str = "device") -> BenchmarkResult:
        model = self._model(ck)
        inputs, outputs = self._tensors(ck, args)
        return model.benchmark(inputs, outputs, warmup_iterations, benchmark_iterations, mode)
