"""The remaining conversion intrinsics as bulk casts (directed rounding to bf16,
float64 -> bf16, the E8M0 scale type, float16) on the GPU against the
reference's vendored headers (fixtures) and the C restatement."""
import os

import numpy as np
import pytest

import oracle
import numba_cuda_b200 as cuda
from numba_cuda_b200 import _lib
from numba_cuda_b200.casts import (cast, cudaRoundMode, cvt_bfloat16raw_to_e8m0, cvt_bfloat16raw_to_fp8,
                                   cvt_double2_to_e8m0x2, cvt_double2_to_fp8x2, cvt_double_to_e8m0,
                                   cvt_double_to_fp8, cvt_e8m0_to_bf16raw, cvt_float2_to_e8m0x2,
                                   cvt_float_to_e8m0, float32_to_bfloat16_rd, float32_to_bfloat16_ru,
                                   float32_to_bfloat16_rz, float64_to_bfloat16, fp8_e8m0_to_float32,
                                   fp8_interpretation_t, saturation_t)

pytestmark = pytest.mark.gpu
RZ, RU, RD = cudaRoundMode.cudaRoundZero, cudaRoundMode.cudaRoundPosInf, cudaRoundMode.cudaRoundMinInf


@pytest.fixture(scope="module")
def gold(golden_dir):
    return np.load(os.path.join(golden_dir, "cast_reference.npz"))


@pytest.mark.parametrize("mode,tag", [(RZ, "rz"), (RU, "ru"), (RD, "rd")])
def test_bf16_directed_rounding(gold, mode, tag):
    x = gold["f32_bits"].view(np.float32)
    got = cast(x, "f32", "bf16", rounding=mode).copy_to_host().view(np.uint16)
    ok = ~np.isnan(x)
    assert (got[ok] == gold[f"bf16_{tag}"][ok]).all()
    assert ((got[~ok] & 0x7FFF) > 0x7F80).all()
    fn = {"rz": float32_to_bfloat16_rz, "ru": float32_to_bfloat16_ru, "rd": float32_to_bfloat16_rd}[tag]
    one = np.float32(1.0) + np.float32(2.0 ** -10)        # between two bf16 values
    assert np.asarray(fn(one)).view(np.uint16) == (0x3F81 if tag == "ru" else 0x3F80)
    assert np.asarray(fn(-one)).view(np.uint16) == (0xBF81 if tag == "rd" else 0xBF80)


def test_float64_to_bfloat16(gold):
    d = gold["f64_inputs"]
    got = cast(d, "f64", "bf16").copy_to_host().view(np.uint16)
    ok = ~np.isnan(d)
    assert (got[ok] == gold["bf16_from_f64"][ok]).all()
    assert ((got[~ok] & 0x7FFF) > 0x7F80).all()
    # double rounding through float32 would give 0x3F80 here; one-step rounding gives 0x3F81
    tricky = np.float64(1.0) + 2.0 ** -8 + 2.0 ** -40
    assert np.asarray(float64_to_bfloat16(tricky)).view(np.uint16) == 0x3F81
    big = np.random.default_rng(4).standard_normal(100003) * 1e3
    assert cast(big, "f64", "bf16").copy_to_host().view(np.uint16).tobytes() == \
        oracle.cast_ex(big, oracle.F64, oracle.BF16).tobytes()


@pytest.mark.parametrize("sat,stag", [(0, "nosat"), (1, "satfinite")])
@pytest.mark.parametrize("mode,mtag", [(RZ, "rz"), (RU, "rp")])
def test_e8m0_encode(gold, sat, stag, mode, mtag):
    x = gold["f32_bits"].view(np.float32)
    got = cast(x, "f32", "e8m0", saturate=sat, rounding=mode).copy_to_host()
    assert (got == gold[f"e8m0_from_f32_{stag}_{mtag}"]).all()
    h = np.arange(65536, dtype=np.uint16)
    got = cast(h, "bf16", "e8m0", saturate=sat, rounding=mode).copy_to_host()
    assert (got == gold[f"e8m0_from_bf16_{stag}_{mtag}"]).all()


def test_e8m0_decode_and_known_answers(gold):
    codes = np.arange(256, dtype=np.uint8)
    assert (cast(codes, "e8m0", "bf16").copy_to_host().view(np.uint16) == gold["e8m0_to_bf16"]).all()
    f = cast(codes, "e8m0", "f32").copy_to_host()
    assert f[127] == 1.0 and f[128] == 2.0 and f[0] == np.float32(2.0 ** -127) and np.isnan(f[255])
    # tests/cudapy/test_fp8_bindings.py:449-560
    assert np.asarray(cvt_e8m0_to_bf16raw(np.uint8(127))).view(np.uint16) == 0x3F80
    over = np.nextafter(np.float32(2.0 ** 127), np.float32(np.inf))
    assert cvt_float_to_e8m0(over, saturation_t.NOSAT, RU) == 0xFF
    assert cvt_float_to_e8m0(over, saturation_t.SATFINITE, RU) == 0xFE
    half = cvt_e8m0_to_bf16raw(np.uint8(126))
    assert cvt_bfloat16raw_to_e8m0(half, saturation_t.NOSAT, RZ) == 126
    assert cvt_bfloat16raw_to_e8m0(half, saturation_t.NOSAT, RU) == 126
    assert fp8_e8m0_to_float32(np.uint8(130)) == 8.0
    with pytest.raises(ValueError):
        cvt_float_to_e8m0(1.0, saturation_t.NOSAT, cudaRoundMode.cudaRoundNearest)


def test_float16_round_trip():
    x = (np.random.default_rng(6).standard_normal(100001) * 100).astype(np.float32)
    x[::1000] = np.inf
    x[1::1000] = 1e-7
    x[2::1000] = 70000.0
    h = cast(x, "f32", "f16").copy_to_host()
    assert h.dtype == np.float16 and h.view(np.uint16).tobytes() == x.astype(np.float16).view(np.uint16).tobytes()
    back = cast(h, "f16", "f32").copy_to_host()
    assert back.tobytes() == h.astype(np.float32).tobytes()


def test_unaligned_and_ragged_inputs():
    x = (np.random.default_rng(7).standard_normal(10007) * 50).astype(np.float32)
    d = cuda.to_device(x)
    for off in (0, 1, 3, 8):
        got = cast(d[off:], "f32", "e8m0", saturate=1, rounding=RU).copy_to_host()
        assert got.tobytes() == oracle.cast_ex(x[off:], oracle.F32, oracle.E8M0, 1, oracle.RU).tobytes()
        got = cast(d[off:], "f32", "bf16", rounding=RD).copy_to_host().view(np.uint16)
        assert got.tobytes() == oracle.cast_ex(x[off:], oracle.F32, oracle.BF16, mode=oracle.RD).tobytes()


def test_unsupported_pairs_raise():
    with pytest.raises(NotImplementedError):
        cast(np.zeros(8, dtype=np.float64), "f64", "f16")
    with pytest.raises(NotImplementedError):
        cast(np.zeros(8, dtype=np.float64), "f64", "e4m3", rounding=RZ)
    with pytest.raises(NotImplementedError):
        cast(np.zeros(8, dtype=np.float32), "f32", "e4m3", rounding=RZ)
    L = _lib.lib()
    assert L.b2k_cast_ex(_lib.FMT_F32, _lib.FMT_BF16, 1, 9, 1024, 2048, 8, None) == _lib.ERR_INVALID_ARG


# ---- float64 and bfloat16 sources of the fp8 / e8m0 encoders ----------------------------
def _doubles_around_fp8():
    """float64 inputs that sit on and next to everything the encoder decides on:
    every fp8 value and every midpoint between neighbours (both formats), each with
    its two float64 neighbours; random magnitudes across and far beyond the fp8
    ranges; random 64-bit patterns (NaNs of both signs, infinities, denormals)."""
    rng = np.random.default_rng(21)
    grid = []
    for fmt in (oracle.E4M3, oracle.E5M2):
        vals = oracle.cast(np.arange(256, dtype=np.uint8), fmt, oracle.F32).astype(np.float64)
        vals = np.unique(vals[np.isfinite(vals)])
        mids = (vals[1:] + vals[:-1]) / 2
        for v in (vals, mids, vals * 1.0625, np.array([464.0, 61440.0, 2.0 ** -10, 2.0 ** -17, 1e300, -1e300])):
            grid += [v, np.nextafter(v, np.inf), np.nextafter(v, -np.inf), -v]
    spread = rng.standard_normal(1 << 19) * np.exp2(rng.uniform(-24, 20, 1 << 19))
    bits = rng.integers(0, 2 ** 64, size=1 << 19, dtype=np.uint64).view(np.float64)
    specials = np.array([0.0, -0.0, np.inf, -np.inf, np.nan, -np.nan, 5e-324, -5e-324])
    return np.concatenate(grid + [spread, bits, specials])


def _want(x, src, dst, sat, mode=oracle.RZ):
    """The reference's own header code where its checker library is there, and the C
    restatement in every case; the two must agree."""
    want = oracle.cast_ex(x, src, dst, sat, mode)
    if oracle.have_ref_headers():
        assert want.tobytes() == oracle.ref_cast(x, src, dst, sat, mode=mode).tobytes()
    return want


@pytest.mark.parametrize("sat", [0, 1])
@pytest.mark.parametrize("fmt,name", [(oracle.E4M3, "e4m3"), (oracle.E5M2, "e5m2")])
def test_float64_to_fp8_is_one_rounding_from_the_double(fmt, name, sat):
    x = _doubles_around_fp8()
    assert x.size > (1 << 20)
    got = cast(x, "f64", name, saturate=sat).copy_to_host()
    want = _want(x, oracle.F64, fmt, sat)
    # integer code on both sides: NaN signs and payload bits included
    assert got.tobytes() == want.tobytes(), np.flatnonzero(got != want)[:8]
    # ragged and unaligned views take the scalar kernel
    d = cuda.to_device(x[:4099])
    for off in (1, 3):
        assert cast(d[off:], "f64", name, saturate=sat).copy_to_host().tobytes() == want[off:4099].tobytes()


def test_float64_to_fp8_differs_from_going_through_float32():
    # just above the midpoint between 1.0 and 1.125 (E4M3): float32 rounds the excess away
    x = np.array([1.0625 + 2.0 ** -40, -(1.0625 + 2.0 ** -40)])
    direct = cast(x, "f64", "e4m3").copy_to_host()
    via = cast(x.astype(np.float32), "f32", "e4m3").copy_to_host()
    assert direct.tolist() == [0x39, 0xB9] and via.tolist() == [0x38, 0xB8]


@pytest.mark.parametrize("sat", [0, 1])
@pytest.mark.parametrize("fmt,name", [(oracle.E4M3, "e4m3"), (oracle.E5M2, "e5m2")])
def test_every_bfloat16_pattern_to_fp8(fmt, name, sat):
    h = np.arange(1 << 16, dtype=np.uint16)
    got = cast(h, "bf16", name, saturate=sat).copy_to_host()
    want = _want(h, oracle.BF16, fmt, sat)
    nan = (h & 0x7FFF) > 0x7F80
    assert got[~nan].tobytes() == want[~nan].tobytes()
    if sat:   # the saturating path is the packed cvt instruction: NaN codes as a class
        assert np.isnan(oracle.cast(got[nan], fmt, oracle.F32)).all()
    else:
        assert got[nan].tobytes() == want[nan].tobytes()


@pytest.mark.parametrize("sat", [0, 1])
@pytest.mark.parametrize("mode", [RZ, RU])
def test_float64_to_e8m0(sat, mode):
    rng = np.random.default_rng(22)
    pow2 = np.exp2(np.arange(-140, 140, dtype=np.float64))
    x = np.concatenate([pow2, np.nextafter(pow2, np.inf), np.nextafter(pow2, 0), -pow2,
                        rng.standard_normal(1 << 18) * np.exp2(rng.uniform(-135, 135, 1 << 18)),
                        rng.integers(0, 2 ** 64, size=1 << 18, dtype=np.uint64).view(np.float64),
                        np.array([0.0, -0.0, np.inf, -np.inf, np.nan, 1e300, 5e-324])])
    got = cast(x, "f64", "e8m0", saturate=sat, rounding=mode).copy_to_host()
    want = _want(x, oracle.F64, oracle.E8M0, sat, int(mode))
    assert got.tobytes() == want.tobytes(), np.flatnonzero(got != want)[:8]


def test_reference_known_answers_for_double_and_bf16raw_sources():
    NOSAT, SAT = saturation_t.NOSAT, saturation_t.SATFINITE
    E4M3, E5M2 = fp8_interpretation_t.E4M3, fp8_interpretation_t.E5M2
    # tests/cudapy/test_fp8_bindings.py:421-447
    assert [int(cvt_double_to_fp8(np.float64(1e300), s, i)) for s, i in
            ((NOSAT, E5M2), (SAT, E5M2), (NOSAT, E4M3), (SAT, E4M3))] == [0x7C, 0x7B, 0x7F, 0x7E]
    # :463-496: 2^127 as a bf16 raw value
    raw = cvt_e8m0_to_bf16raw(np.uint8(254))
    assert [int(cvt_bfloat16raw_to_fp8(raw, s, i)) for s, i in
            ((NOSAT, E5M2), (SAT, E5M2), (NOSAT, E4M3), (SAT, E4M3))] == [0x7C, 0x7B, 0x7F, 0x7E]
    # :521-539
    over = np.nextafter(np.float64(2.0 ** 127), np.float64(np.inf))
    assert cvt_double_to_e8m0(over, NOSAT, RU) == 0xFF and cvt_double_to_e8m0(over, SAT, RU) == 0xFE
    # the two-element forms put x[0] in the low byte
    assert cvt_double2_to_fp8x2((1.0, -2.0), SAT, E4M3) == 0x38 | (0xC0 << 8)
    assert cvt_float2_to_e8m0x2((1.0, 4.0), SAT, RZ) == 127 | (129 << 8)
    assert cvt_double2_to_e8m0x2((0.5, 3.0), SAT, RU) == 126 | (129 << 8)
    if oracle.have_ref_headers():
        R = oracle.ref_headers()
        assert cvt_double2_to_fp8x2((0.3, 1e9), NOSAT, E5M2) == R.ref_cvt_double2_to_fp8x2(0.3, 1e9, 0, 1)
        assert cvt_float2_to_e8m0x2((0.3, 1e9), NOSAT, RU) == R.ref_cvt_float2_to_e8m0x2(0.3, 1e9, 0, 2)
        assert cvt_double2_to_e8m0x2((0.3, 1e9), SAT, RZ) == R.ref_cvt_double2_to_e8m0x2(0.3, 1e9, 1, 1)
