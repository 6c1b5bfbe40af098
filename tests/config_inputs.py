"""Seeded synthetic inputs of the benchmark configurations, exactly as they are
defined: NumPy ``default_rng`` streams drawn in a fixed order.  Test helper."""
import queue
import threading

import numpy as np

C5_CHUNK = 1 << 26
C5_CHUNKS = 16
NAN_BITS = 0x7FC00000


def c5_specials() -> np.ndarray:
    s = np.array([np.inf, -np.inf, 0.0, 1e6, -1e6], dtype=np.float32)
    s[2:3] = np.array([NAN_BITS], dtype=np.uint32).view(np.float32)
    return s


def c5_chunks(chunks: int = C5_CHUNKS, chunk: int = C5_CHUNK):
    """Configuration 5: 2^30 float32 values, normal(0, 4), about 1 % of the positions
    overwritten by +inf, -inf, NaN (bits 0x7FC00000), +1e6, -1e6 in turn.  ONE generator,
    ``default_rng(3)``, used in this order chunk by chunk (the chunked procedure is the
    definition): ``4 * standard_normal(chunk)``, then ``random(chunk) < 0.01`` as the
    mask, then the specials cycling on from where the previous chunk stopped.  Yields
    ``(index, array)``; the arrays are produced by a background thread one chunk ahead
    (the draws release the GIL), in order."""
    specials = c5_specials()
    q: "queue.Queue" = queue.Queue(maxsize=2)

    def produce():
        rng = np.random.default_rng(3)
        placed = 0
        for k in range(chunks):
            xc = np.float32(4.0) * rng.standard_normal(chunk, dtype=np.float32)
            mc = rng.random(chunk, dtype=np.float32) < 0.01
            count = int(mc.sum())
            xc[mc] = specials[(placed + np.arange(count)) % 5]
            placed += count
            q.put((k, xc))
        q.put(None)

    threading.Thread(target=produce, daemon=True).start()
    while True:
        item = q.get()
        if item is None:
            return
        yield item


def c3_normals(rows: int, cols: int) -> np.ndarray:
    """Configuration 3: ``default_rng(2).standard_normal((rows, cols), float32)``."""
    return np.random.default_rng(2).standard_normal((rows, cols), dtype=np.float32)


def block_checksums(a: np.ndarray, rows_per_block: int = 4096) -> np.ndarray:
    """Three 64-bit checksums of the BIT PATTERNS of every block of ``rows_per_block`` rows of
    a 2-D float array: xor, wrap-around sum, and wrap-around sum weighted by position (odd
    weights, so that two values changing places show).  Shape ``(blocks, 3)``, uint64."""
    rows = a.shape[0]
    assert rows % rows_per_block == 0
    bits = np.ascontiguousarray(a).view(np.uint32 if a.dtype.itemsize == 4 else np.uint64)
    bits = bits.reshape(rows // rows_per_block, -1).astype(np.uint64)
    weights = (np.arange(bits.shape[1], dtype=np.uint64) << np.uint64(1)) | np.uint64(1)
    with np.errstate(over="ignore"):
        return np.stack([np.bitwise_xor.reduce(bits, axis=1), np.add.reduce(bits, axis=1, dtype=np.uint64),
                         np.add.reduce(bits * weights, axis=1, dtype=np.uint64)], axis=1)
