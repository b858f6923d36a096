"""Native compiler backend: C++ tensor-IR pass pipeline (csrc/compiler) with tiling /
placement / fusion knobs, a text-in / text-out `nkipy-b200-opt` driver, a CPU execution
oracle and CUDA code generation — the counterpart of the reference's `nkigen` package."""

from . import apis, transforms
from .control_flow import LoopIndex, fori_loop
from .execution import run_ir, verify_against_numpy
from .knob import knob
from .trace import TracedArray, trace
from .transforms import apply_complete_knob_pipeline, apply_passes


def __getattr__(name):
    if name == "CustomOp":
        from .custom_op import CustomOp

        return CustomOp
    raise AttributeError(name)


__all__ = ["trace", "TracedArray", "CustomOp", "verify_against_numpy", "run_ir", "apply_passes",
           "apply_complete_knob_pipeline", "apis", "transforms", "knob", "fori_loop", "LoopIndex"]
