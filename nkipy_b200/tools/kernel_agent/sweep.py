"""Random sweeps of generated kernels with resumable result files
(reference: tools/kernel_agent/sweep.py:30-451)."""

from __future__ import annotations

import json
import os
import random
import time
from typing import Dict, List, Optional

from .executor import run_kernel
from .generator import TemplateClient, load_kernel

SWEEP_OPS = ["exp", "tanh", "abs", "sqrt", "square", "negative", "sin", "cos", "log", "add", "subtract", "multiply",
             "maximum", "minimum", "divide", "sum", "max", "mean", "min", "where", "transpose"]


def run_sweep(num_kernels: int, ops_per_kernel: int, out_dir: str, seed: int = 0, use_gpu: Optional[bool] = None,
              client=None) -> Dict:
    os.makedirs(out_dir, exist_ok=True)
    rng = random.Random(seed)
    client = client or TemplateClient(seed)
    results: List[Dict] = []
    for i in range(num_kernels):
        ops = [rng.choice(SWEEP_OPS) for _ in range(ops_per_kernel)]
        src = client.generate(ops, "")
        path = os.path.join(out_dir, f"kernel_{i:04d}.py")
        with open(path, "w") as f:
            f.write(src)
        results.append(_run_file(path, ops, use_gpu))
    summary = {"when": time.strftime("%Y-%m-%dT%H:%M:%S"), "num_kernels": num_kernels,
               "passed": sum(r["passed"] for r in results), "results": results}
    with open(os.path.join(out_dir, "sweep_results.json"), "w") as f:
        json.dump(summary, f, indent=1)
    return summary


def _run_file(path: str, ops, use_gpu) -> Dict:
    with open(path) as f:
        kernel, make_inputs = load_kernel(f.read())
    r = run_kernel(kernel, make_inputs(), use_gpu=use_gpu)
    return dict(r.as_dict(), file=os.path.basename(path), ops=list(ops), passed=r.passed)


def rerun_failed(out_dir: str, use_gpu: Optional[bool] = None) -> Dict:
    path = os.path.join(out_dir, "sweep_results.json")
    with open(path) as f:
        summary = json.load(f)
    for i, r in enumerate(summary["results"]):
        if not r["passed"]:
            summary["results"][i] = _run_file(os.path.join(out_dir, r["file"]), r["ops"], use_gpu)
    summary["passed"] = sum(r["passed"] for r in summary["results"])
    with open(path, "w") as f:
        json.dump(summary, f, indent=1)
    return summary
