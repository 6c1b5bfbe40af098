"""Seeded inputs for the conversions with an integer side (fp8 value types from and
to integers, bf16 from and to integers): the generator of the committed fixture and
the tests build the same arrays from these functions."""
import numpy as np

INT_NAMES = ("int8", "int16", "int32", "int64", "uint8", "uint16", "uint32", "uint64")


def integers(name: str, n: int = 4096, seed: int = 11) -> np.ndarray:
    """``n`` random values whose bit lengths cover the whole type, followed by the
    edge cases: 0, the ends of the range, and every power of two with its two
    neighbours, in both signs where the type has one."""
    dt = np.dtype(name)
    info = np.iinfo(dt)
    rng = np.random.default_rng(seed + dt.itemsize + (100 if dt.kind == "u" else 0))
    mags = rng.integers(0, 2 ** 63, n, dtype=np.uint64) >> rng.integers(0, 64, n).astype(np.uint64)
    flip = rng.random(n) < 0.5
    vals = [int(m) for m in mags]
    if dt.kind == "i":
        vals = [-v if f else v for v, f in zip(vals, flip)]
    edge = [0, info.max, info.min, info.max - 1, info.min + 1]
    edge += [(1 << k) + d for k in range(dt.itemsize * 8 + 1) for d in (-1, 0, 1)]
    vals += edge + [-e for e in edge]
    return np.array([min(max(v, info.min), info.max) for v in vals], dtype=dt)


def bf16_patterns() -> np.ndarray:
    """Every 16th bfloat16 bit pattern plus everything near the integer ranges' ends,
    halves (for ties), zeros, infinities and NaNs."""
    base = np.arange(0, 65536, 16, dtype=np.uint32)
    near = []
    for e in (0, 1, 126, 127, 128, 133, 134, 135, 141, 142, 143, 157, 158, 159, 189, 190, 191, 254, 255):
        for m in (0, 1, 2, 63, 64, 65, 126, 127):
            for s in (0, 1):
                near.append((s << 15) | (e << 7) | m)
    halves = [((s << 15) | ((127 + k) << 7) | m) for k in range(0, 9) for m in range(128) for s in (0, 1)]
    return np.unique(np.concatenate([base, np.array(near + halves, dtype=np.uint32)])).astype(np.uint16)
