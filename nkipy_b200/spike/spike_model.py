"""Loaded kernel with named-tensor validation, automatic output allocation and
benchmarking (spike/src/spike/spike_model.py:1-363 in the reference)."""

from __future__ import annotations

import json
import os
import statistics
import time
from dataclasses import dataclass, field
from typing import Dict, List, Optional

import numpy as np

from ..core.dtypes import dtype_from_name
from .spike_singleton import get_spike_singleton
from .spike_tensor import SpikeTensor


@dataclass
class BenchmarkResult:
    mean_ms: float
    min_ms: float
    max_ms: float
    std_dev_ms: float
    iterations: int
    warmup_iterations: int
    durations_ms: List[float] = field(default_factory=list)

    def __str__(self):
        return (f"mean {self.mean_ms:.4f} ms, min {self.min_ms:.4f} ms, max {self.max_ms:.4f} ms, "
                f"std {self.std_dev_ms:.4f} ms over {self.iterations} iterations ({self.warmup_iterations} warm-up)")


def _result(durations: List[float], warmup: int) -> BenchmarkResult:
    return BenchmarkResult(statistics.fmean(durations), min(durations), max(durations),
                           statistics.pstdev(durations) if len(durations) > 1 else 0.0, len(durations), warmup,
                           durations)


def _parse_exec_durations(events_json: str) -> List[float]:
    """Device durations (ms) of each execute from `kernel_exec` start/stop pairs keyed by tracking id."""
    events = json.loads(events_json)["events"]
    start: Dict[int, float] = {}
    out = []
    for e in events:
        if e["event_type"] != "kernel_exec":
            continue
        if e["phase"] == "start":
            start[e["tracking_id"]] = e["device_timestamp_ns"]
        elif e["tracking_id"] in start:
            out.append((e["device_timestamp_ns"] - start.pop(e["tracking_id"])) / 1e6)
    return out


class SpikeModel:
    def __init__(self, model_ref, name: str, neff_path: str):
        self.model_ref = model_ref
        self.name = name
        self.neff_path = neff_path
        info = get_spike_singleton().get_tensor_info(model_ref)
        self.input_info = dict(info.inputs)
        self.output_info = dict(info.outputs)
        self.input_order = list(info.input_order)
        self.output_order = list(info.output_order)
        self.aliases = dict(info.aliases)

    @classmethod
    def load_from_neff(cls, neff_path: str, name: Optional[str] = None, core_id: int = 0, cc_enabled: bool = False,
                       rank_id: int = 0, world_size: int = 1):
        """Load a compiled kernel (a cubin with its `.json` plan next to it)."""
        if not os.path.exists(neff_path):
            raise FileNotFoundError(neff_path)
        ref = get_spike_singleton().load_model(str(neff_path), core_id, cc_enabled, rank_id, world_size)
        model = cls(ref, name or ref.name, str(neff_path))
        if ref.has_collectives and ref.collective_world > 1:
            model._attach_collective_workspace(rank_id, world_size)
        return model

    def _attach_collective_workspace(self, rank_id: int, world_size: int) -> None:
        """Collectives inside the module run over a symmetric workspace: one allocation per rank mapped into every
        rank.  It is made here, at load time, over the process group of the job (every rank loads the same module
        at the same point of the program), and its addresses go to the C++ module as the peer table."""
        from ..parallel.comm import TPGroup
        from ..parallel.symm import SymmetricMemory

        tp = TPGroup.from_env()
        if tp.world_size != world_size or tp.rank != rank_id:
            raise RuntimeError(f"module with collectives over {world_size} ranks loaded as rank {rank_id}, but the "
                               f"process group says rank {tp.rank} of {tp.world_size}")
        self._cc_mem = SymmetricMemory(tp, int(self.model_ref.workspace_bytes))
        self.model_ref.set_collective_workspace([int(p) for p in self._cc_mem.ptrs])

    load_from_cubin = load_from_neff

    # ------------------------------------------------------------------ tensors
    def allocate_output_tensors(self, core_id: int = 0) -> Dict[str, SpikeTensor]:
        out = {}
        for nm in self.output_order:
            m = self.output_info[nm]
            out[nm] = SpikeTensor.empty(tuple(m.shape), dtype_from_name(m.dtype), nm, core_id)
        return out

    def _validate_io(self, tensors: Dict[str, SpikeTensor], expected, kind: str) -> None:
        missing = [n for n in expected if n not in tensors]
        extra = [n for n in tensors if n not in expected]
        if missing or extra:
            raise ValueError(f"{kind} tensors of '{self.name}' do not match: missing {missing}, unexpected {extra}; "
                             f"expected {list(expected)}")
        for nm, m in expected.items():
            t = tensors[nm]
            if tuple(t.shape) != tuple(m.shape):
                raise ValueError(f"{kind} '{nm}': expected shape {tuple(m.shape)}, got {tuple(t.shape)}")
            if np.dtype(t.dtype) != dtype_from_name(m.dtype) and not (
                    m.dtype == "u8" and np.dtype(t.dtype) == np.bool_):
                raise ValueError(f"{kind} '{nm}': expected dtype {m.dtype}, got {t.dtype}")
            if t.core_id != self.model_ref.core_id:
                raise ValueError(f"{kind} '{nm}' lives on core {t.core_id}, model on core {self.model_ref.core_id}")

    def __call__(self, inputs: Dict[str, SpikeTensor], outputs: Optional[Dict[str, SpikeTensor]] = None,
                 save_trace: bool = False, ntff_name: Optional[str] = None):
        """Run the kernel.  Without `outputs` they are allocated and returned as a dict."""
        self._validate_io(inputs, self.input_info, "input")
        auto = outputs is None
        if auto:
            outputs = self.allocate_output_tensors(self.model_ref.core_id)
        self._validate_io(outputs, self.output_info, "output")
        if save_trace and not ntff_name:
            ntff_name = os.path.splitext(self.neff_path)[0] + ".trace.json"
        get_spike_singleton().execute(self.model_ref, {k: v.tensor_ref for k, v in inputs.items()},
                                      {k: v.tensor_ref for k, v in outputs.items()}, ntff_name or "", save_trace)
        return outputs if auto else None

    # ------------------------------------------------------------------ benchmark
    def benchmark(self, inputs: Dict[str, SpikeTensor], outputs: Optional[Dict[str, SpikeTensor]] = None,
                  warmup_iterations: int = 5, benchmark_iterations: int = 100, mode: str = "device") -> BenchmarkResult:
        if outputs is None:
            outputs = self.allocate_output_tensors(self.model_ref.core_id)
        if mode == "device":
            from .spike_singleton import _native

            with _native().SystemTraceSession(self.model_ref.core_id) as session:
                for _ in range(warmup_iterations):
                    self(inputs, outputs)
                session.drain_events()
                for _ in range(benchmark_iterations):
                    self(inputs, outputs)
                durations = _parse_exec_durations(session.fetch_events_json())
            return _result(durations, warmup_iterations)
        if mode == "host":
            for _ in range(warmup_iterations):
                self(inputs, outputs)
            durations = []
            for _ in range(benchmark_iterations):
                t0 = time.perf_counter()
                self(inputs, outputs)
                durations.append((time.perf_counter() - t0) * 1e3)
            return _result(durations, warmup_iterations)
        raise ValueError("mode must be 'device' or 'host'")

    def unload(self) -> None:
        """Collective for modules with collectives (the symmetric workspace is released by all ranks together)."""
        get_spike_singleton().unload_model(self.model_ref)
        mem = getattr(self, "_cc_mem", None)
        if mem is not None:
            self._cc_mem = None
            mem.close()
