"""Smallest end-to-end use of the tracing frontend: `A.T @ B` on 1024 x 1024 fp16 matrices
(reference: examples/playground/simple_nkipy_kernel.py:30-132).

The function is plain NumPy.  Called directly it runs on the CPU; wrapped in `baremetal_jit` it is
traced once, lowered to CUDA C++ (the matmul becomes a tcgen05 GEMM), compiled with nvcc, loaded by the
C++ runtime and executed on the GPU.  `BaremetalExecutor.benchmark` times the loaded kernel.
"""
import os
import sys

import numpy as np

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", ".."))


def matmul_kernel(a, b):
    return a.T @ b


def main():
    import torch

    rng = np.random.default_rng(0)
    a = rng.standard_normal((1024, 1024)).astype(np.float16)
    b = rng.standard_normal((1024, 1024)).astype(np.float16)
    want = matmul_kernel(a.astype(np.float32), b.astype(np.float32))
    if not torch.cuda.is_available():
        got = matmul_kernel(a, b)
        print("no GPU: ran in CPU direct mode, max |err| =", float(np.abs(got.astype(np.float32) - want).max()))
        return 0
    from nkipy_b200.core.compile import compile_to_neff, trace
    from nkipy_b200.runtime import BaremetalExecutor, CompiledKernel, baremetal_jit

    got = baremetal_jit(matmul_kernel)(a, b)
    rel = float(np.abs(got.astype(np.float32) - want).max() / np.abs(want).max())
    print(f"baremetal_jit: max rel err vs fp32 NumPy = {rel:.2e}")
    assert rel < 2e-2
    # the same kernel compiled once and timed on the device
    traced = trace(matmul_kernel)
    traced.specialize(a, b)
    cubin = compile_to_neff(traced, neff_name="matmul_kernel.cubin")
    with BaremetalExecutor() as ex:
        stats = ex.benchmark(CompiledKernel(traced, cubin), a, b, warmup_iterations=5, benchmark_iterations=50)
        print("benchmark:", stats)
    return 0


if __name__ == "__main__":
    sys.exit(main())
