"""Hand-written kernels inside programs traced with the nkigen front end (nkigen/nkigen/custom_op.py:42-228 in the
reference: a decorator that turns a kernel-builder function into an op with declared operand and result specs).

    @custom_op(input_specs=[((128, 256), "f32")], output_specs=[((128, 256), "f32")], grid=(128,), block=(256,),
               reference=lambda x: x * 2)
    def double(input_specs, output_specs):
        return 'extern "C" __global__ void double(const float* x, float* y) { ... }'

    y = double(x)          # a custom_call node while tracing; the reference on NumPy arrays
"""

from ..core.cuda_op import CudaCustomOp as CustomOp, cuda_custom_op  # noqa: F401
from ..core.nki_op import NKICustomOpHandle, nki_custom_op


def custom_op(*, input_specs, output_specs, **launch):
    """Decorator form of `nki_custom_op(kernel_builder=...)`; the entry point defaults to the function's name."""

    def deco(builder) -> NKICustomOpHandle:
        launch.setdefault("name", builder.__name__)
        return nki_custom_op(kernel_builder=builder, input_specs=input_specs, output_specs=output_specs, **launch)

    return deco
