"""bf16 conversion API (the conversion subset of numba/cuda/bf16.py:204-269:
floating-point and integer conversions in the four rounding modes, bit casts),
host-callable and bulk."""
from . import casts as _casts
from .casts import (bfloat16_as_int16, bfloat16_as_uint16, bfloat16_to_float32, cast,  # noqa: F401
                    float32_to_bfloat16, float32_to_bfloat16_rd, float32_to_bfloat16_rn,
                    float32_to_bfloat16_ru, float32_to_bfloat16_rz, float64_to_bfloat16,
                    int16_as_bfloat16, uint16_as_bfloat16)
from .devicearray import bfloat16_dtype  # noqa: F401

for _name in _casts._BF16_INT_NAMES:   # int16_to_bfloat16_rn ... bfloat16_to_uint64_ru, bfloat16_to_int8_rz
    globals()[_name] = getattr(_casts, _name)
del _name
