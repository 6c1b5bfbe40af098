"""fp8 conversion API (the conversion subset of numba.cuda.fp8 /
numba/cuda/_internal/cuda_fp8.py), host-callable and bulk."""
from .casts import (cast, cudaRoundMode, cvt_bfloat16raw_to_e8m0, cvt_bfloat16raw_to_fp8,  # noqa: F401
                    cvt_double2_to_e8m0x2, cvt_double2_to_fp8x2, cvt_double_to_e8m0, cvt_double_to_fp8,
                    cvt_e8m0_to_bf16raw, cvt_float2_to_e8m0x2, cvt_float2_to_fp8x2, cvt_float_to_e8m0,
                    cvt_float_to_fp8, fp8_e4m3, fp8_e4m3_to, fp8_e4m3_to_float32, fp8_e5m2, fp8_e5m2_to,
                    fp8_e5m2_to_float32, fp8_e8m0, fp8_e8m0_to, fp8_e8m0_to_float32, fp8_interpretation_t,
                    fp8x2_e4m3, fp8x2_e5m2, fp8x2_e8m0, fp8x2_to, fp8x4_e4m3, fp8x4_e5m2, fp8x4_e8m0, fp8x4_to,
                    saturation_t)
