"""Random sweeps of generated kernels.

Every iteration generates one kernel, runs it through numpy -> compile -> device (or the IR interpreter
where there is no device) and appends one JSON line to ``sweep_<utc time>.jsonl`` -- flushed at once, so
a sweep that is stopped or dies keeps what it found.  An iteration that runs longer than `timeout` seconds
is abandoned (SIGALRM) and recorded as failed at stage "timeout"; SIGINT / SIGTERM finish the iteration in
flight, write the summary and return.  `run_rerun` replays the kernels of an earlier log from their saved
source, `rerun_failed` only the failed ones of a sweep directory.
(reference: nkipy/src/nkipy/tools/kernel_agent/sweep.py:30-451 -- the record fields and the
stop / timeout behaviour follow it; generation is offline by default here.)
"""

from __future__ import annotations

import contextlib
import dataclasses
import json
import os
import random
import signal
import threading
import time
from datetime import datetime, timezone
from typing import Any, Callable, Dict, Iterable, List, Optional

from .executor import ExecutionResult, run_kernel
from .generator import TemplateClient, load_kernel

SWEEP_OPS = ["exp", "tanh", "abs", "sqrt", "square", "negative", "sin", "cos", "log", "add", "subtract", "multiply",
             "maximum", "minimum", "divide", "sum", "max", "mean", "min", "where", "transpose"]


@dataclasses.dataclass
class SweepRecord:
    """One line of a sweep log."""

    iteration: int
    timestamp: str
    prompt: str = ""
    model_id: str = "template"
    kernel_name: str = ""
    file: str = ""
    ops: List[str] = dataclasses.field(default_factory=list)
    generated_code: str = ""
    input_specs: Dict[str, Any] = dataclasses.field(default_factory=dict)
    numpy_success: Optional[bool] = None
    numpy_error: Optional[str] = None
    compile_success: Optional[bool] = None
    compile_error: Optional[str] = None
    hardware_success: Optional[bool] = None       # None: no device, the interpreter checked the graph instead
    hardware_error: Optional[str] = None
    max_diff: Optional[float] = None
    allclose: Optional[bool] = None
    passed: bool = False
    failure_stage: Optional[str] = None
    error_message: Optional[str] = None
    duration_seconds: float = 0.0
    rerun_source: Optional[str] = None

    def as_dict(self) -> Dict[str, Any]:
        return dataclasses.asdict(self)

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "SweepRecord":
        names = {f.name for f in dataclasses.fields(cls)}
        return cls(**{k: v for k, v in d.items() if k in names})

    def absorb(self, r: ExecutionResult) -> None:
        """Copy the outcome of the three-stage executor into the record."""
        self.numpy_success, self.compile_success = r.numpy_ok, (r.compile_ok if r.numpy_ok else None)
        self.hardware_success = r.hardware_ok
        self.max_diff, self.allclose = r.max_abs_err, r.numerics_ok
        self.passed, self.failure_stage = r.passed, r.error_stage
        self.error_message = r.error
        if r.error_stage in ("numpy", "compile", "hardware"):
            setattr(self, f"{r.error_stage}_error", r.error)


class _IterationTimeout(Exception):
    pass


class _Stop:
    """Set by SIGINT / SIGTERM; the sweep loop looks at it between iterations."""

    def __init__(self):
        self.requested = False
        self.signum: Optional[int] = None


@contextlib.contextmanager
def _sweep_signals(stop: _Stop):
    """Handlers for the duration of a sweep; the previous ones come back afterwards.  Outside the main
    thread Python allows no handlers: the sweep then runs without timeout and without graceful stop."""
    if threading.current_thread() is not threading.main_thread():
        yield False
        return

    def on_stop(signum, frame):
        stop.requested, stop.signum = True, signum

    def on_alarm(signum, frame):
        raise _IterationTimeout()

    prev = {s: signal.signal(s, h) for s, h in
            ((signal.SIGINT, on_stop), (signal.SIGTERM, on_stop), (signal.SIGALRM, on_alarm))}
    try:
        yield True
    finally:
        signal.alarm(0)
        for s, h in prev.items():
            signal.signal(s, h)


def _utc() -> str:
    return datetime.now(timezone.utc).strftime("%Y-%m-%dT%H:%M:%SZ")


def _stamp() -> str:
    return datetime.now(timezone.utc).strftime("%Y%m%d_%H%M%S_%f")


def _input_specs(inputs: Iterable) -> Dict[str, Any]:
    out = {}
    for i, a in enumerate(inputs):
        shape = getattr(a, "shape", None)
        out[f"arg{i}"] = {"shape": list(shape) if shape is not None else None,
                          "dtype": str(getattr(a, "dtype", type(a).__name__))}
    return out


def _execute(record: SweepRecord, body: Callable[[SweepRecord], None], log, fail_counts: Dict[str, int],
             timeout: int, armed: bool) -> None:
    """Run one iteration body under the alarm, finish the record and append it to the log."""
    t0 = time.time()
    try:
        if armed and timeout > 0:
            signal.alarm(int(timeout))
        body(record)
    except _IterationTimeout:
        record.passed, record.failure_stage = False, "timeout"
        record.error_message = f"iteration exceeded {timeout} s"
    except Exception as e:       # generation or loading failed: the executor reports its own stages itself
        record.passed, record.failure_stage = False, record.failure_stage or "generate"
        record.error_message = f"{type(e).__name__}: {e}"
    finally:
        if armed:
            signal.alarm(0)
    record.duration_seconds = round(time.time() - t0, 3)
    if not record.passed:
        stage = record.failure_stage or "unknown"
        fail_counts[stage] = fail_counts.get(stage, 0) + 1
    log.write(json.dumps(record.as_dict()) + "\n")
    log.flush()


def _run_source(record: SweepRecord, source: str, use_gpu: Optional[bool]) -> None:
    kernel, make_inputs = load_kernel(source)
    record.kernel_name = getattr(kernel, "__name__", "kernel")
    inputs = make_inputs()
    record.input_specs = _input_specs(inputs)
    record.absorb(run_kernel(kernel, inputs, use_gpu=use_gpu))


def _summary_line(done: int, passed: int, fail_counts: Dict[str, int], t0: float) -> str:
    fails = ", ".join(f"{k}: {v}" for k, v in sorted(fail_counts.items())) or "none"
    return f"[{done} kernels, {time.time() - t0:.0f} s] passed {passed}, failed by stage: {fails}"


def _finish(out_dir: str, log_path: str, records: List[SweepRecord], fail_counts, stop: _Stop, name: str) -> Dict:
    results = [dict(r.as_dict(), hardware_ok=r.hardware_success) for r in records]
    summary = {"when": _utc(), "log": log_path, "num_kernels": len(records),
               "passed": sum(r.passed for r in records), "failed_by_stage": dict(fail_counts),
               "interrupted": stop.requested, "results": results}
    with open(os.path.join(out_dir, name), "w") as f:
        json.dump(summary, f, indent=1)
    return summary


def run_sweep(num_kernels: Optional[int], ops_per_kernel: int, out_dir: str, seed: int = 0,
              use_gpu: Optional[bool] = None, client=None, timeout: int = 120, delay: float = 0.0,
              summary_interval: int = 10, verbose: bool = False) -> Dict:
    """Generate and test `num_kernels` kernels (None: until SIGINT / SIGTERM).  Returns the summary, which is
    also written to ``sweep_results.json``; ``summary["log"]`` names the JSONL log."""
    os.makedirs(out_dir, exist_ok=True)
    rng = random.Random(seed)
    client = client or TemplateClient(seed)
    model_id = getattr(client, "model_id", type(client).__name__)
    log_path = os.path.join(out_dir, f"sweep_{_stamp()}.jsonl")
    records: List[SweepRecord] = []
    fail_counts: Dict[str, int] = {}
    stop, t0 = _Stop(), time.time()
    with _sweep_signals(stop) as armed, open(log_path, "a") as log:
        i = 0
        while (num_kernels is None or i < num_kernels) and not stop.requested:
            ops = [rng.choice(SWEEP_OPS) for _ in range(ops_per_kernel)]
            rec = SweepRecord(iteration=i, timestamp=_utc(), ops=ops, model_id=model_id,
                              prompt="ops: " + ", ".join(ops), file=f"kernel_{i:04d}.py")

            def body(r: SweepRecord, ops=ops):
                r.generated_code = client.generate(ops, "")
                with open(os.path.join(out_dir, r.file), "w") as f:
                    f.write(r.generated_code)
                _run_source(r, r.generated_code, use_gpu)

            _execute(rec, body, log, fail_counts, timeout, armed)
            records.append(rec)
            i += 1
            if verbose and summary_interval and i % summary_interval == 0:
                print(_summary_line(i, sum(r.passed for r in records), fail_counts, t0), flush=True)
            if delay and not stop.requested:
                time.sleep(delay)
    return _finish(out_dir, log_path, records, fail_counts, stop, "sweep_results.json")


def load_records(path: str) -> List[SweepRecord]:
    """The records of a JSONL sweep log (lines that do not parse, such as a torn last line, are skipped)."""
    out = []
    with open(path) as f:
        for line in f:
            line = line.strip()
            if not line:
                continue
            try:
                out.append(SweepRecord.from_dict(json.loads(line)))
            except (ValueError, TypeError):
                continue
    return out


def run_rerun(source_path: str, use_gpu: Optional[bool] = None, out_dir: Optional[str] = None, timeout: int = 120,
              only_failed: bool = False, summary_interval: int = 10, verbose: bool = False) -> Dict:
    """Execute again the kernels saved in a JSONL log of an earlier sweep (their source is in the log, nothing is
    generated).  Writes ``rerun_<utc time>.jsonl`` and ``rerun_results.json`` to `out_dir` (default: beside the
    source) and returns the summary."""
    if not os.path.exists(source_path):
        raise FileNotFoundError(f"sweep log not found: {source_path}")
    if not source_path.endswith(".jsonl"):
        raise ValueError(f"a sweep log is a .jsonl file, got {os.path.basename(source_path)!r}")
    out_dir = out_dir or os.path.dirname(os.path.abspath(source_path))
    os.makedirs(out_dir, exist_ok=True)
    sources = [r for r in load_records(source_path) if r.generated_code and not (only_failed and r.passed)]
    log_path = os.path.join(out_dir, f"rerun_{_stamp()}.jsonl")
    records: List[SweepRecord] = []
    fail_counts: Dict[str, int] = {}
    stop, t0 = _Stop(), time.time()
    with _sweep_signals(stop) as armed, open(log_path, "a") as log:
        for n, old in enumerate(sources):
            if stop.requested:
                break
            rec = SweepRecord(iteration=old.iteration, timestamp=_utc(), ops=list(old.ops), model_id=old.model_id,
                              prompt=old.prompt, file=old.file, generated_code=old.generated_code,
                              rerun_source=os.path.basename(source_path))
            _execute(rec, lambda r: _run_source(r, r.generated_code, use_gpu), log, fail_counts, timeout, armed)
            records.append(rec)
            if verbose and summary_interval and (n + 1) % summary_interval == 0:
                print(_summary_line(n + 1, sum(r.passed for r in records), fail_counts, t0), flush=True)
    return _finish(out_dir, log_path, records, fail_counts, stop, "rerun_results.json")


def rerun_failed(out_dir: str, use_gpu: Optional[bool] = None, timeout: int = 120) -> Dict:
    """Re-run the failed kernels recorded in ``sweep_results.json`` of a sweep directory and update that file."""
    path = os.path.join(out_dir, "sweep_results.json")
    with open(path) as f:
        summary = json.load(f)
    stop, fail_counts = _Stop(), {}
    log_path = os.path.join(out_dir, f"rerun_{_stamp()}.jsonl")
    with _sweep_signals(stop) as armed, open(log_path, "a") as log:
        for i, r in enumerate(summary["results"]):
            if r["passed"] or stop.requested:
                continue
            with open(os.path.join(out_dir, r["file"])) as f:
                source = f.read()
            rec = SweepRecord(iteration=r.get("iteration", i), timestamp=_utc(), ops=list(r.get("ops", [])),
                              file=r["file"], generated_code=source, rerun_source="sweep_results.json")
            _execute(rec, lambda x: _run_source(x, x.generated_code, use_gpu), log, fail_counts, timeout, armed)
            summary["results"][i] = dict(rec.as_dict(), hardware_ok=rec.hardware_success)
    summary["passed"] = sum(r["passed"] for r in summary["results"])
    with open(path, "w") as f:
        json.dump(summary, f, indent=1)
    return summary
