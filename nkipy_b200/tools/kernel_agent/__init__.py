"""kernel_agent: discover which NumPy operations trace, compile and run, test generated kernels through
the three stages numpy -> compile -> device, and sweep randomly composed kernels
(counterpart of nkipy/src/nkipy/tools/kernel_agent in the reference)."""

import dataclasses as _dc
import os as _os

from .executor import ExecutionResult, compare, gpu_available, run_kernel  # noqa: E402,F401
from .generator import BedrockClient, TemplateClient, load_kernel, system_prompt  # noqa: E402,F401
from .ops import TARGET_OPS, all_ops, build_kernel, discover, test_op  # noqa: E402,F401
from .sweep import SweepRecord, load_records, rerun_failed, run_rerun, run_sweep  # noqa: E402,F401


@_dc.dataclass
class StageResult:
    """Outcome of one pipeline stage (numpy / compile / hardware)."""
    stage: str
    ok: bool
    error: str = ""


def stages(result: ExecutionResult):
    """An `ExecutionResult` as a list of `StageResult`s."""
    out = [StageResult("numpy", result.numpy_ok), StageResult("compile", result.compile_ok)]
    if result.hardware_ok is not None:
        out.append(StageResult("hardware", bool(result.hardware_ok)))
    if result.error_stage:
        for s in out:
            if s.stage == result.error_stage:
                s.error = result.error or ""
    return out


# names of the reference's module-level API
get_all_ops = all_ops
discover_ops = discover
make_kernel = build_kernel


def generate_kernel(ops, client=None, prompt: str = "") -> str:
    return (client or TemplateClient()).generate(list(ops), prompt)


def build_inputs(source: str, seed: int = 0):
    return load_kernel(source)[1](seed)


def compile_code(source: str):
    """Trace + lower the kernel of a generated source; returns the CUDA C++ text."""
    from nkipy_b200.compiler.codegen import lower_to_cuda
    from nkipy_b200.core.compile import trace

    kernel, make_inputs = load_kernel(source)
    return lower_to_cuda(trace(kernel).specialize(*make_inputs()))


def get_kernel_prompts():
    d = _os.path.join(_os.path.dirname(_os.path.abspath(__file__)), "prompts")
    return {f[:-4]: open(_os.path.join(d, f)).read() for f in sorted(_os.listdir(d)) if f.endswith(".txt")}


KERNEL_PROMPTS = get_kernel_prompts()
