"""Compile driver: traced kernel -> CUDA C++ -> nvcc -> cubin + launch plan.

API of the reference's nkipy.core.compile (nkipy/src/nkipy/core/compile.py:22-384) with
the Neuron compiler replaced by this package's code generator and nvcc:

    trace(fn, backend)             -> NKIPyKernel
    compile_to_neff(kernel, out)   -> path of the compiled artifact (alias compile_to_cubin)
    lower_to_nki(kernel, *args)    -> generated kernel source (alias lower_to_cuda)
    Compiler(CompilationConfig).compile_in_directory(...)
    CompilationTarget, get_platform_target, nkipy_compiler_args, _get/_set_build_dir

The artifact is ``<name>.cubin`` with ``<name>.json`` (the plan) beside it; with
``save_artifacts`` the IR text and the generated ``.cu`` are kept too.  A failing nvcc run
raises `CompilationError` carrying the command line, stdout and stderr.
"""

from __future__ import annotations

import enum
import os
import shlex
import shutil
import subprocess
import tempfile
from dataclasses import dataclass
from pathlib import Path
from typing import Optional

from .ir import Graph
from .trace import NKIPyKernel, trace

__all__ = ["trace", "Compiler", "CompilationConfig", "CompilationResult", "CompilationTarget", "CompilationError",
           "get_platform_target", "get_ir", "compile_to_neff", "compile_to_cubin", "lower_to_nki", "lower_to_cuda",
           "nkipy_compiler_args", "DEFAULT_ADDITIONAL_COMPILER_ARGS", "NKIPY_KERNEL_ADDITIONAL_COMPILER_ARGS",
           "_get_build_dir", "_set_build_dir"]

_build_dir = os.environ.get("NKIPY_B200_BUILD_DIR", "/tmp/nkipy_b200_build")
KERNELS_DIR = Path(__file__).resolve().parents[2] / "csrc" / "kernels"

DEFAULT_ADDITIONAL_COMPILER_ARGS = "-O3"
NKIPY_KERNEL_ADDITIONAL_COMPILER_ARGS = "-O3 --use_fast_math"
nkipy_compiler_args = DEFAULT_ADDITIONAL_COMPILER_ARGS


def _get_build_dir() -> str:
    return _build_dir


def _set_build_dir(path: str) -> None:
    global _build_dir
    _build_dir = str(path)


class CompilationTarget(enum.Enum):
    SM100A = "sm_100a"
    DEFAULT = "default"
    # names of the reference's targets resolve to the one device this framework serves
    TRN1 = "sm_100a-compat-trn1"
    TRN2 = "sm_100a-compat-trn2"
    TRN3 = "sm_100a-compat-trn3"


def get_platform_target() -> CompilationTarget:
    return CompilationTarget.SM100A


class CompilationError(RuntimeError):
    def __init__(self, message: str, command=None, stdout: str = "", stderr: str = ""):
        super().__init__(message)
        self.command, self.stdout, self.stderr = command, stdout, stderr


@dataclass
class CompilationConfig:
    target: CompilationTarget = CompilationTarget.DEFAULT
    additional_args: str = ""
    save_artifacts: bool = False
    use_tcgen05: bool = True
    in_process: bool = False      # accepted for parity; nvcc always runs as a subprocess


@dataclass
class CompilationResult:
    neff_path: str
    plan_path: str
    work_dir: str
    source_path: Optional[str] = None

    @property
    def cubin_path(self) -> str:
        return self.neff_path


def get_ir(kernel: NKIPyKernel) -> Graph:
    if kernel._code is None:
        raise RuntimeError("kernel has not been specialized; call kernel.specialize(*args) first")
    return kernel._code


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise CompilationError("nvcc not found; set NVCC or install the CUDA toolkit")


class Compiler:
    def __init__(self, config: Optional[CompilationConfig] = None):
        self.config = config or CompilationConfig()

    def _command(self, src: Path, out: Path) -> list:
        extra = shlex.split(self.config.additional_args) if self.config.additional_args else []
        if not any(a.startswith("-O") for a in extra):
            extra = ["-O3"] + extra
        return [_nvcc(), "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-cubin",
                f"-I{KERNELS_DIR}", *extra, str(src), "-o", str(out)]

    def compile_graph(self, graph: Graph, work_dir: str, output_file: str = "kernel.cubin") -> CompilationResult:
        from ..compiler.codegen import generate

        work = Path(work_dir)
        work.mkdir(parents=True, exist_ok=True)
        stem = Path(output_file).stem
        program = generate(graph, use_tcgen05=self.config.use_tcgen05)
        src = work / f"{stem}.cu"
        out = work / output_file
        plan = work / f"{stem}.json"
        src.write_text(program.source)
        if self.config.save_artifacts:
            (work / f"{stem}.ir.txt").write_text(graph.to_text())
        cmd = self._command(src, out)
        cwd = os.getcwd()
        try:
            res = subprocess.run(cmd, capture_output=True, text=True, cwd=str(work))
        finally:
            os.chdir(cwd)
        if res.returncode != 0:
            raise CompilationError(
                f"nvcc failed with exit code {res.returncode}\ncommand: {' '.join(cmd)}\nstderr:\n{res.stderr}\n"
                f"stdout:\n{res.stdout}", cmd, res.stdout, res.stderr)
        if not out.exists():
            raise CompilationError(
                f"{out.name} was expected but not generated by nvcc although it exited 0\ncommand: {' '.join(cmd)}\n"
                f"stderr:\n{res.stderr}\nstdout:\n{res.stdout}", cmd, res.stdout, res.stderr)
        plan.write_text(program.plan_json())
        if not self.config.save_artifacts:
            src.unlink(missing_ok=True)
        return CompilationResult(str(out), str(plan), str(work), str(src) if self.config.save_artifacts else None)

    def compile_in_directory(self, ir: Graph, output_dir: Optional[str] = None, output_file: str = "kernel.cubin"
                             ) -> CompilationResult:
        if output_dir is None:
            output_dir = tempfile.mkdtemp(prefix="nkipy_b200_")
        return self.compile_graph(ir, output_dir, output_file)


def compile_to_neff(kernel, output_dir: Optional[str] = None, neff_name: str = "kernel.cubin",
                    additional_compiler_args: str = "", save_artifacts: bool = False,
                    target: CompilationTarget = CompilationTarget.DEFAULT, use_tcgen05: bool = True) -> str:
    """Compile a specialized kernel (or a `Graph`); returns the path of the cubin."""
    ir = kernel if isinstance(kernel, Graph) else get_ir(kernel)
    if neff_name.endswith(".neff"):
        neff_name = neff_name[:-5] + ".cubin"
    if getattr(kernel, "backend", None) == "nkigen":
        # kernels traced for the native backend go through its pass pipeline first: tiling knobs, fusion
        # groups and the shared-memory budget decide what the code generator emits
        from ..nkigen.transforms import apply_complete_knob_pipeline

        ir = Graph.from_text(apply_complete_knob_pipeline(ir.to_text()))
    cfg = CompilationConfig(target, additional_compiler_args, save_artifacts, use_tcgen05)
    return Compiler(cfg).compile_in_directory(ir, output_dir or _get_build_dir(), neff_name).neff_path


compile_to_cubin = compile_to_neff


def lower_to_nki(kernel, *args, **kwargs) -> str:
    """Generated kernel source for `kernel` specialized on `args` (CUDA C++ here)."""
    from ..compiler.codegen import lower_to_cuda as _lower

    if isinstance(kernel, Graph):
        return _lower(kernel)
    if not isinstance(kernel, NKIPyKernel):
        kernel = NKIPyKernel(kernel, "hlo")
    if args or kwargs or kernel._code is None:
        kernel.specialize(*args, **kwargs)
    return _lower(kernel._code)


lower_to_cuda = lower_to_nki
