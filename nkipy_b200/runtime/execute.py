"""One-shot trace -> compile -> load -> run helpers
(nkipy/src/nkipy/runtime/execute.py:25-163 in the reference).

`baremetal_run_traced_kernel(kernel, *args)` compiles without caching (the build
directory of the kernel is wiped first), uploads the array arguments, lets aliased outputs
share their input's device buffer, materialises zero-element outputs on the host, writes
mutated inputs back into the caller's arrays and filters the automatically appended
alias outputs from the returned values.
"""

from __future__ import annotations

import os
import shutil
from typing import Optional

import numpy as np

from ..core.compile import CompilationTarget, _get_build_dir, compile_to_neff, trace
from ..core.dtypes import sanitize_dtype
from ..core.ir import prepare_io_mapping
from ..core.trace import NKIPyKernel
from .device_kernel import DeviceKernel
from .device_tensor import DeviceTensor


def _compile_kernel(kernel: NKIPyKernel, *args, artifacts_dir: Optional[str] = None,
                    additional_compiler_args: str = "", target=CompilationTarget.DEFAULT, **kwargs):
    ir = kernel.specialize(*args, **kwargs)
    build_dir = artifacts_dir or os.path.join(_get_build_dir(), f"{kernel.__name__}_jit")
    if os.path.isdir(build_dir):
        shutil.rmtree(build_dir)
    neff = compile_to_neff(ir, build_dir, f"{kernel.__name__}.cubin",
                           additional_compiler_args=additional_compiler_args,
                           save_artifacts=artifacts_dir is not None, target=target)
    return ir, neff


def _execute_neff(ir, neff_path: str, arrays, save_trace: bool = False):
    """arrays: user ndarrays in parameter order."""
    names = [p.original_name.replace(".must_alias_input", "") for p in ir.inputs]
    originals = {n: a for n, a in zip(names, arrays)}
    in_placeholders = ir.inputs
    for p in in_placeholders:
        p.original_name = p.name.replace(".must_alias_input", "")
    input_arrays, alias_names = prepare_io_mapping(in_placeholders, ir.aliases, originals)
    model = DeviceKernel.load_from_neff(neff_path)
    try:
        inputs = {n: DeviceTensor.from_numpy(np.ascontiguousarray(a.astype(sanitize_dtype(a.dtype), copy=False)), n)
                  for n, a in input_arrays.items()}
        outputs, host_outputs = {}, {}
        for i, o in enumerate(ir.outputs):
            if int(np.prod(o.shape, dtype=np.int64)) == 0:
                host_outputs[o.name] = np.zeros(o.shape, dtype=o.dtype)       # nothing to compute on the device
                outputs[o.name] = DeviceTensor.empty(o.shape, o.dtype, o.name)
            elif i in alias_names:
                outputs[o.name] = inputs[alias_names[i]]                      # shares the input buffer
            else:
                outputs[o.name] = DeviceTensor.empty(o.shape, o.dtype, o.name)
        model(inputs, outputs, save_trace=save_trace)
        results = []
        for i, o in enumerate(ir.outputs):
            val = host_outputs.get(o.name)
            if val is None:
                val = outputs[o.name].numpy()
            if i in alias_names:
                src_name = alias_names[i].replace(".must_alias_input", "")
                np.copyto(originals[src_name], val.astype(originals[src_name].dtype, copy=False))
            if i not in ir.auto_aliased_indices:
                results.append(val)
    finally:
        model.unload()
    if not results:
        return None
    return results[0] if len(results) == 1 else tuple(results)


def baremetal_run_traced_kernel(kernel, *args, artifacts_dir: Optional[str] = None, save_trace: bool = False,
                                additional_compiler_args: str = "", target=CompilationTarget.DEFAULT, **kwargs):
    if not isinstance(kernel, NKIPyKernel):
        kernel = trace(kernel)
    ir, neff = _compile_kernel(kernel, *args, artifacts_dir=artifacts_dir,
                               additional_compiler_args=additional_compiler_args, target=target, **kwargs)
    arrays = [a for a in args if isinstance(a, np.ndarray)] + [v for v in kwargs.values() if isinstance(v, np.ndarray)]
    return _execute_neff(ir, neff, arrays, save_trace=save_trace)
