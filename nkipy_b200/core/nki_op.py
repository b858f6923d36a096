from .cuda_op import *  # noqa: F401,F403
from .cuda_op import (CudaCustomOp, NKICustomOp, NKICustomOpHandle, NKIOp, cuda_custom_op, nki_custom_op,  # noqa: F401
                      wrap_nki_kernel)

CUDA_AVAILABLE = True          # the custom-op frontend itself needs no toolchain until compile time
BETA3_COMPILE_MODES = ()       # no alternative kernel frontends on this target
