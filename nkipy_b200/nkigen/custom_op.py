"""Hand-written kernels inside traced programs (nkigen/nkigen/custom_op.py:42-228 and
nkipy/src/nkipy/core/nki_op.py in the reference).  See `nkipy_b200.core.cuda_op`."""

from ..core.cuda_op import CudaCustomOp as CustomOp, cuda_custom_op  # noqa: F401
