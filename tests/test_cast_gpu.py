"""bf16 / fp8 bulk casts on the GPU against the reference's vendored-header
arithmetic (fixtures from tests/golden/make_golden.py, the C restatement, and
the known-answer bytes of numba/cuda/tests/cudapy/test_fp8_bindings.py)."""
import os

import numpy as np
import pytest
import torch

import oracle
import numba_cuda_b200 as cuda
from numba_cuda_b200 import _lib
from numba_cuda_b200.casts import (cast, cvt_float2_to_fp8x2, cvt_float_to_fp8, fp8_e4m3, fp8_e4m3_to_float32,
                                   fp8_e5m2, fp8_e5m2_to_float32, fp8_interpretation_t, saturation_t,
                                   float32_to_bfloat16, bfloat16_to_float32)

pytestmark = pytest.mark.gpu
E4M3, E5M2 = fp8_interpretation_t.E4M3, fp8_interpretation_t.E5M2
NOSAT, SATFINITE = saturation_t.NOSAT, saturation_t.SATFINITE


@pytest.fixture(scope="module")
def gold(golden_dir):
    return np.load(os.path.join(golden_dir, "cast_reference.npz"))


def is_nan_code(codes, fmt):
    mag = codes & 0x7F
    return mag == 0x7F if fmt == "e4m3" else mag > 0x7C


@pytest.mark.parametrize("fmt", ["e4m3", "e5m2"])
@pytest.mark.parametrize("sat", [1, 0])
def test_encode_matches_reference_headers(gold, fmt, sat):
    x = gold["f32_bits"].view(np.float32)
    want = gold[f"{fmt}_{'satfinite' if sat else 'nosat'}"]
    got = cast(x, "f32", fmt, saturate=sat).copy_to_host()
    nan_in = np.isnan(x)
    assert (got[~nan_in] == want[~nan_in]).all()
    # NaN inputs: a NaN code on both sides; positive quiet NaN gives exactly 0x7F
    assert is_nan_code(got[nan_in], fmt).all() and is_nan_code(want[nan_in], fmt).all()
    qnan = np.array([0x7FC00000], dtype=np.uint32).view(np.float32)
    assert cast(qnan, "f32", fmt, saturate=sat).copy_to_host()[0] == 0x7F


@pytest.mark.parametrize("fmt", ["e4m3", "e5m2"])
def test_decode_all_codes(gold, fmt):
    codes = np.arange(256, dtype=np.uint8)
    got = cast(codes, fmt, "f32").copy_to_host()
    want = gold[f"{fmt}_decode_f32_bits"].view(np.float32)
    nan = np.isnan(want)
    assert (np.isnan(got) == nan).all()
    assert got[~nan].tobytes() == want[~nan].tobytes()
    # encode(decode(code)) is the identity on every finite code; E5M2 infinities
    # survive without saturation and clamp to the largest finite code with it
    fin = np.isfinite(want)
    back = cast(got, "f32", fmt, saturate=1).copy_to_host()
    assert (back[fin] == codes[fin]).all()
    back0 = cast(got, "f32", fmt, saturate=0).copy_to_host()
    assert (back0[~nan] == codes[~nan]).all()
    inf = np.isinf(want)
    assert ((back[inf] & 0x7F) == 0x7B).all()


def test_bf16_encode_matches_reference_headers(gold):
    x = gold["f32_bits"].view(np.float32)
    got = cast(x, "f32", "bf16").copy_to_host().view(np.uint16)
    want = gold["bf16_rn"]
    nan_in = np.isnan(x)
    assert (got[~nan_in] == want[~nan_in]).all()
    assert ((got[nan_in] & 0x7FFF) > 0x7F80).all()
    qnan = np.array([0x7FC00000], dtype=np.uint32).view(np.float32)
    assert cast(qnan, "f32", "bf16").copy_to_host().view(np.uint16)[0] == 0x7FFF


def test_bf16_decode_all_patterns():
    h = np.arange(1 << 16, dtype=np.uint16)
    got = cast(h, "bf16", "f32").copy_to_host()
    want = oracle.cast(h, oracle.BF16, oracle.F32)
    nan = np.isnan(want)
    assert (np.isnan(got) == nan).all()
    assert got[~nan].tobytes() == want[~nan].tobytes()
    # quiet NaNs keep their payload; signalling ones may be quieted by the convert instruction
    quiet = nan & ((h & 0x0040) != 0)
    assert got[quiet].tobytes() == want[quiet].tobytes()


def test_known_answer_bytes():
    # test_fp8_bindings.py:388-419
    assert cvt_float_to_fp8(1e20, NOSAT, E5M2) == 0x7C
    assert cvt_float_to_fp8(1e20, SATFINITE, E5M2) == 0x7B
    assert cvt_float_to_fp8(1e20, NOSAT, E4M3) == 0x7F
    assert cvt_float_to_fp8(1e20, SATFINITE, E4M3) == 0x7E
    # exact small values round-trip (:88-128, :334-349); NaN stays NaN (:162-177)
    for v in (1.0, 2.0, 4.0, -1.0, 0.5):
        assert fp8_e4m3_to_float32(fp8_e4m3(v)) == v
        assert fp8_e5m2_to_float32(fp8_e5m2(v)) == v
    assert np.isnan(fp8_e4m3_to_float32(fp8_e4m3(float("nan"))))
    assert np.isnan(fp8_e5m2_to_float32(fp8_e5m2(float("nan"))))
    # spot values of the vendored header
    for v, code in ((448.0, 0x7E), (464.0, 0x7E), (465.0, 0x7E), (1e6, 0x7E), (float("inf"), 0x7E),
                    (float("-inf"), 0xFE), (2.0 ** -10, 0x00), (0.017, 0x09)):
        assert fp8_e4m3(v) == code, v
    # packed pair: first element in the low byte (cuda_fp8.hpp:291-313)
    assert cvt_float2_to_fp8x2((1.0, 2.0), SATFINITE, E4M3) == (0x40 << 8) | 0x38
    # bf16: 1.5 is exact (test_bfloat16.py:518-529)
    assert bfloat16_to_float32(float32_to_bfloat16(1.5)) == 1.5
    assert float(bfloat16_to_float32(float32_to_bfloat16(3.14))) == float(np.float32(3.140625))


def config5_chunk(n, seed=3):
    """Configuration-5 generator for one chunk: normal(0, 4) with ~1 % specials."""
    rng = np.random.default_rng(seed)
    x = np.float32(4.0) * rng.standard_normal(n, dtype=np.float32)
    m = rng.random(n, dtype=np.float32) < 0.01
    specials = np.array([np.inf, -np.inf, np.nan, 1e6, -1e6], dtype=np.float32)
    specials[2:3] = np.array([0x7FC00000], dtype=np.uint32).view(np.float32)
    x[m] = specials[np.arange(int(m.sum())) % 5]
    return x


@pytest.mark.parametrize("n", [0, 1, 3, 4, 5, 1023, 4096, (1 << 22) + 3])
def test_config5_distribution_round_trips(n):
    x = config5_chunk(n)
    d = cuda.to_device(x) if n else x
    for fmt, code in (("e4m3", oracle.E4M3), ("e5m2", oracle.E5M2)):
        e = cast(d, "f32", fmt)
        want_codes = oracle.cast(x, oracle.F32, code, 1)
        assert e.copy_to_host().tobytes() == want_codes.tobytes()
        back = cast(e, fmt, "f32").copy_to_host()
        want_back = oracle.cast(want_codes, code, oracle.F32)
        nan = np.isnan(want_back)
        assert (np.isnan(back) == nan).all() and back[~nan].tobytes() == want_back[~nan].tobytes()
    b = cast(d, "f32", "bf16")
    want_b = oracle.cast(x, oracle.F32, oracle.BF16)
    assert b.copy_to_host().view(np.uint16).tobytes() == want_b.tobytes()
    back = cast(b, "bf16", "f32").copy_to_host()
    assert back.tobytes() == oracle.cast(want_b, oracle.BF16, oracle.F32).tobytes()


@pytest.mark.skipif(not oracle.have_ref_headers(), reason="reference-header checker not present")
def test_against_reference_headers_on_random_bits():
    bits = np.random.default_rng(17).integers(0, 2 ** 32, size=1 << 20, dtype=np.uint32)
    x = bits.view(np.float32)
    ok = ~np.isnan(x)
    for fmt, code in (("e4m3", oracle.E4M3), ("e5m2", oracle.E5M2)):
        for sat in (0, 1):
            got = cast(x, "f32", fmt, saturate=sat).copy_to_host()
            want = oracle.ref_cast(x, oracle.F32, code, sat)
            assert (got[ok] == want[ok]).all(), (fmt, sat)
    got = cast(x, "f32", "bf16").copy_to_host().view(np.uint16)
    assert (got[ok] == oracle.ref_cast(x, oracle.F32, oracle.BF16)[ok]).all()


def test_unaligned_views_use_the_scalar_kernel():
    x = config5_chunk(10007)
    d = cuda.to_device(x)
    for off in (1, 2, 3, 4, 5, 8, 12):          # 4 and 12: 16- but not 32-byte aligned (128-bit path)
        got = cast(d[off:], "f32", "e4m3").copy_to_host()
        assert got.tobytes() == oracle.cast(x[off:], oracle.F32, oracle.E4M3, 1).tobytes()
    codes = cuda.to_device(oracle.cast(x, oracle.F32, oracle.E4M3, 1))
    want = oracle.cast(oracle.cast(x, oracle.F32, oracle.E4M3, 1), oracle.E4M3, oracle.F32)
    for off in (1, 2, 3, 4, 8, 12):
        got = cast(codes[off:], "e4m3", "f32").copy_to_host()
        nan = np.isnan(want[off:])
        assert got[~nan].tobytes() == want[off:][~nan].tobytes()


def test_bf16_paths_by_alignment():
    x = config5_chunk(20011)
    d = cuda.to_device(x)
    want = oracle.cast(x, oracle.F32, oracle.BF16)
    hb = cuda.to_device(want)
    for off in (0, 1, 4, 8, 16):
        got = cast(d[off:], "f32", "bf16").copy_to_host().view(np.uint16)
        assert got.tobytes() == want[off:].tobytes(), off
        back = cast(hb[off:], "bf16", "f32").copy_to_host()
        assert back.tobytes() == oracle.cast(want[off:], oracle.BF16, oracle.F32).tobytes(), off


def test_out_argument_shapes_and_errors():
    x = config5_chunk(4096).reshape(64, 64)
    out = cuda.device_array((64, 64), dtype=np.uint8)
    ret = cast(x, "f32", "e4m3", out=out)
    assert ret is out and ret.shape == (64, 64)
    with pytest.raises(ValueError):
        cast(x, "f32", "e4m3", out=cuda.device_array(100, dtype=np.uint8))
    with pytest.raises(TypeError):
        cast(x.astype(np.float64), "f32", "e4m3")
    with pytest.raises(NotImplementedError):
        cast(np.zeros(16, dtype=np.uint8), "e4m3", "e5m2")


def test_negative_nan_encoding_is_a_nan():
    neg = np.array([0xFFC00000, 0xFF800001, 0xFFFFFFFF], dtype=np.uint32).view(np.float32)
    for fmt in ("e4m3", "e5m2"):
        for sat in (0, 1):
            got = cast(neg, "f32", fmt, saturate=sat).copy_to_host()
            assert is_nan_code(got, fmt).all()
    # the non-saturating path follows the header's host algorithm: sign dropped, 0x7F
    assert (cast(neg, "f32", "e4m3", saturate=0).copy_to_host() == 0x7F).all()
