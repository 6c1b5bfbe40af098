"""fp8 conversion API (the conversion subset of numba.cuda.fp8 /
numba/cuda/_internal/cuda_fp8.py), host-callable and bulk."""
from .casts import (cast, cvt_float2_to_fp8x2, cvt_float_to_fp8, fp8_e4m3, fp8_e4m3_to_float32,  # noqa: F401
                    fp8_e5m2, fp8_e5m2_to_float32, fp8_interpretation_t, saturation_t)
