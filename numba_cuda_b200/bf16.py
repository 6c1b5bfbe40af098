"""bf16 conversion API (the conversion subset of numba/cuda/bf16.py:204-207),
host-callable and bulk."""
from .casts import bfloat16_to_float32, cast, float32_to_bfloat16, float32_to_bfloat16_rn  # noqa: F401
from .devicearray import bfloat16_dtype  # noqa: F401
