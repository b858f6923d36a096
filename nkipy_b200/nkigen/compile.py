"""Native-backend compile entry (nkigen/nkigen/compile.py:16-74 in the reference):
IR text -> pass pipeline -> CUDA C++ -> nvcc -> cubin + plan."""

from __future__ import annotations

from typing import Optional

from ..core.compile import CompilationConfig, Compiler
from ..core.ir import Graph
from .transforms import apply_complete_knob_pipeline


def compile_to_neff(ir_text_or_kernel, output_dir: str, neff_name: str = "kernel.cubin", target: str = "sm_100a",
                    dump_dir: Optional[str] = None, additional_compiler_args: str = "",
                    save_artifacts: bool = False) -> str:
    ir_text = ir_text_or_kernel if isinstance(ir_text_or_kernel, str) else ir_text_or_kernel.to_ir()
    lowered = apply_complete_knob_pipeline(ir_text, target=target, dump_dir=dump_dir)
    graph = Graph.from_text(lowered)
    cfg = CompilationConfig(additional_args=additional_compiler_args, save_artifacts=save_artifacts)
    return Compiler(cfg).compile_graph(graph, output_dir, neff_name).neff_path


compile_to_cubin = compile_to_neff
