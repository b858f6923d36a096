"""A hand-written CUDA kernel used as an operation of a traced program
(reference: examples/playground/simple_nki_kernel.py:20-125 does the same with an `@nki.jit` kernel).

The custom op adds two 128 x 512 fp32 tensors.  Inside a traced function the call becomes a
`custom_call` node whose source is compiled into the same module as the generated kernels; on plain
NumPy arrays the reference implementation runs.
"""
import os
import sys

import numpy as np

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", ".."))

from nkipy_b200.core.cuda_op import cuda_custom_op  # noqa: E402

SRC = r"""
extern "C" __global__ void tensor_add_kernel(const float* a, const float* b, float* out) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < 128 * 512) out[i] = a[i] + b[i];
}
"""

tensor_add = cuda_custom_op("tensor_add", SRC, "tensor_add_kernel", [((128, 512), "f32")], grid=(256,), block=(256,),
                            reference=lambda a, b: a + b)


def kernel(a, b):
    return tensor_add(a, b) * 2.0


def main():
    import torch

    rng = np.random.default_rng(0)
    a = rng.standard_normal((128, 512)).astype(np.float32)
    b = rng.standard_normal((128, 512)).astype(np.float32)
    want = (a + b) * 2.0
    if torch.cuda.is_available():
        from nkipy_b200.runtime import baremetal_jit

        got = baremetal_jit(kernel)(a, b)
        where = "gpu"
    else:
        got = kernel(a, b)
        where = "cpu reference"
    err = float(np.abs(np.asarray(got) - want).max())
    print(f"custom op on {where}: max |err| = {err:.2e}")
    assert err < 1e-5
    return 0


if __name__ == "__main__":
    sys.exit(main())
