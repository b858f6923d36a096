"""Driver of the native pass pipeline (the role of nkigen/nkigen/transforms/nkipy_opt.py).

`apply_complete_knob_pipeline(ir_text, ...)` runs the default pipeline through the
`nkipy-b200-opt` binary (a subprocess, text in / text out, like the reference's batches of
C++ passes) followed by the in-process Python stage ``py:ir-to-cuda`` when a CUDA source is
requested.  `stop_after` accepts a 1-based index, a pass name, ``name:N`` or a group name
(`PASS_GROUPS`); `dump_dir` receives ``NN_<pass>.ir`` after every stage, numbered
continuously across the native and the Python stages.  A failing run raises
``RuntimeError`` carrying the command, stdout and stderr.
"""

from __future__ import annotations

import os
import subprocess
from typing import List, Optional, Sequence

from ..compiler.native import build, opt_path

PY_PASSES = ["py:ir-to-cuda"]


def _native():
    import importlib

    try:
        return importlib.import_module("nkipy_b200.nkigen._b200c")
    except ImportError:
        build()
        return importlib.import_module("nkipy_b200.nkigen._b200c")


def pass_list() -> List[str]:
    return [p[0] for p in _native().list_passes() if p[1] != "oracle"] + PY_PASSES


def _groups():
    groups = {}
    for name, group, _ in _native().list_passes():
        groups.setdefault(group, []).append(name)
    groups["codegen"] = list(PY_PASSES)
    return groups


PASS_GROUPS = None


def pass_groups():
    global PASS_GROUPS
    if PASS_GROUPS is None:
        PASS_GROUPS = _groups()
    return PASS_GROUPS


def run_opt(ir_text: str, args: Sequence[str]) -> str:
    """One `nkipy-b200-opt` invocation; raises RuntimeError with command + output on failure."""
    if not opt_path().exists():
        build()
    cmd = [str(opt_path()), *args, "-"]
    res = subprocess.run(cmd, input=ir_text, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"nkipy-b200-opt failed (exit {res.returncode})\ncommand: {' '.join(cmd)}\n"
                           f"stderr:\n{res.stderr}\nstdout:\n{res.stdout}")
    return res.stdout


def apply_passes(ir_text: str, passes: Sequence[str], in_process: bool = True, **options) -> str:
    """Run the named native passes in order."""
    if in_process:
        return _native().apply_passes(ir_text, list(passes), **options)
    args = []
    for p in passes:
        args += ["--pass", p]
    for k, v in options.items():
        if k == "fast_math":
            if v:
                args.append("--fast-math")
        else:
            args += [f"--{k.replace('_', '-')}", str(v)]
    return run_opt(ir_text, args)


def apply_complete_knob_pipeline(ir_text: str, target: str = "sm_100a", dump_dir: Optional[str] = None,
                                 stop_after=None, smem_capacity: Optional[int] = None, fast_math: bool = False,
                                 emit_cuda: bool = False):
    """Default pipeline.  Returns the final IR text, or (ir_text, cuda_source) with emit_cuda."""
    native = [p for p in pass_list() if not p.startswith("py:")]
    stop = "" if stop_after is None else str(stop_after)
    run_py = emit_cuda
    if stop:
        if stop.isdigit():
            if int(stop) > len(native):
                if int(stop) > len(native) + len(PY_PASSES):
                    raise ValueError(f"stop_after index {stop} out of range")
                stop, run_py = "", True
        elif stop in PY_PASSES or stop == "codegen":
            stop, run_py = "", True
        else:
            run_py = False
    args = ["--pipeline", "--target", target]
    if stop:
        args += ["--stop-after", stop]
    if dump_dir:
        os.makedirs(dump_dir, exist_ok=True)
        args += ["--dump-dir", dump_dir]
    if smem_capacity is not None:
        args += ["--smem-capacity", str(smem_capacity)]
    if fast_math:
        args.append("--fast-math")
    out = run_opt(ir_text, args)
    if not run_py:
        return out
    from ..compiler.codegen import generate
    from ..core.ir import Graph

    program = generate(Graph.from_text(out))
    if dump_dir:
        idx = len(native) + 1
        with open(os.path.join(dump_dir, f"{idx:02d}_py_ir-to-cuda.cu"), "w") as f:
            f.write(program.source)
    return out, program.source
