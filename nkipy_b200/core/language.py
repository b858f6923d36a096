"""Extra element types usable in kernels (nkipy/src/nkipy/core/language.py:5-9)."""
import ml_dtypes

bfloat16 = ml_dtypes.bfloat16
float8_e5m2 = ml_dtypes.float8_e5m2
float8_e4m3 = ml_dtypes.float8_e4m3fn
