"""Every public name a user of the reference imports (nkipy/src/nkipy/__init__.py, core/*/__init__.py,
runtime/__init__.py, spike/src/spike/__init__.py, nkigen/src/nkigen/__init__.py, tools/kernel_agent/__init__.py)
has a counterpart at the same place in this package."""
import importlib

import pytest

SURFACE = {
 "nkipy_b200": "knob",
 "nkipy_b200.core.trace": "NKIPyKernel",
 "nkipy_b200.core.compile": "trace Compiler CompilationConfig CompilationResult CompilationTarget get_platform_target get_ir compile_to_neff lower_to_nki nkipy_compiler_args DEFAULT_ADDITIONAL_COMPILER_ARGS NKIPY_KERNEL_ADDITIONAL_COMPILER_ARGS _get_build_dir _set_build_dir",
 "nkipy_b200.core.ops": "Op get_backend set_source_location",
 "nkipy_b200.core.tensor": "NKIPyTensorRef TensorArithmeticMixin TensorOperationMixin find_source_loc",
 "nkipy_b200.core.tensor_apis": "constant topk rms_norm softmax conv2d conv3d zeros full",
 "nkipy_b200.core.backend": "TensorPlaceholder AliasInfo ComputationIR prepare_io_mapping tracing get_backend set_source_location",
 "nkipy_b200.core.backend.hlo": "HLOModule HLOOp HLOTensor HLOTraceContext get_hlo_context find_common_type_hlo scalar_dtype_hlo",
 "nkipy_b200.core.backend.nkigen": "NkiGenTensor NkiGenTraceContext NkiGenIR get_nkigen_context",
 "nkipy_b200.core.knob": "knob",
 "nkipy_b200.core.nki_op": "wrap_nki_kernel NKICustomOp nki_custom_op NKICustomOpHandle NKIOp BETA3_COMPILE_MODES",
 "nkipy_b200.core.specs": "ShapeSpec TypeSpec InputSpec ScalarInputSpec TensorInputSpec KernelSpec CommonTypes",
 "nkipy_b200.core.language": "bfloat16 float8_e5m2 float8_e4m3",
 "nkipy_b200.core.typing": "tensor mutable_tensor mutable immutable",
 "nkipy_b200.core.logger": "get_logger",
 "nkipy_b200.distributed.collectives": "all_gather all_reduce reduce_scatter all_to_all",
 "nkipy_b200.runtime": "baremetal_jit baremetal_run_traced_kernel BaremetalExecutor CompiledKernel DeviceKernel DeviceTensor is_neuron_compatible",
 "nkipy_b200.tools.kernel_agent": "run_kernel ExecutionResult StageResult TARGET_OPS get_all_ops test_op discover_ops make_kernel generate_kernel build_inputs compile_code run_sweep run_rerun SweepRecord get_kernel_prompts KERNEL_PROMPTS",
 "nkipy_b200.spike": "SpikeModel SpikeTensor SpikeProfiler configure reset get_spike_singleton NrtError SpikeError SystemTraceSession BenchmarkResult ModelTensorInfo NrtModel NrtTensor TensorMetadata",
 "nkipy_b200.nkigen": "trace TracedArray CustomOp verify_against_numpy apply_passes apis transforms knob",
}


@pytest.mark.parametrize("module", sorted(SURFACE))
def test_public_names_exist(module):
    m = importlib.import_module(module)
    missing = [n for n in SURFACE[module].split() if not hasattr(m, n)]
    assert not missing, (module, missing)


def test_op_registry_size():
    import nkipy_b200.core.ops as o

    assert sum(isinstance(getattr(o, n), o.Op) for n in dir(o)) >= 111     # core/ops/__init__.py:180-306
