"""bf16 conversion API (the conversion subset of numba/cuda/bf16.py:204-210),
host-callable and bulk."""
from .casts import (bfloat16_to_float32, cast, float32_to_bfloat16, float32_to_bfloat16_rd,  # noqa: F401
                    float32_to_bfloat16_rn, float32_to_bfloat16_ru, float32_to_bfloat16_rz,
                    float64_to_bfloat16)
from .devicearray import bfloat16_dtype  # noqa: F401
