"""Conversions with an integer side on the GPU: the fp8 value types' constructors
from, and conversion operators to, every numeric type; the packed x2 / x4 types;
bf16 from and to integers in the four rounding modes.  Checked bit for bit against
the CPU restatement (itself pinned to the reference's headers) and the fixture the
reference's headers produced."""
import os

import numpy as np
import pytest

import oracle
import numba_cuda_b200 as cuda
from numba_cuda_b200 import _lib, bf16 as b16
from numba_cuda_b200.casts import (cast, cudaRoundMode, fp8_e4m3, fp8_e4m3_to, fp8_e5m2, fp8_e5m2_to, fp8_e8m0,
                                   fp8_e8m0_to, fp8x2_e4m3, fp8x2_e8m0, fp8x2_to, fp8x4_e4m3, fp8x4_e5m2,
                                   fp8x4_to)
from value_type_inputs import INT_NAMES, bf16_patterns, integers

pytestmark = pytest.mark.gpu
FORMATS = {"e4m3": oracle.E4M3, "e5m2": oracle.E5M2, "e8m0": oracle.E8M0}
INTS = {name: getattr(oracle, "I" + name[3:] if name.startswith("int") else "U" + name[4:]) for name in INT_NAMES}
MODES = {"rn": (cudaRoundMode.cudaRoundNearest, oracle.RN), "rz": (cudaRoundMode.cudaRoundZero, oracle.RZ),
         "ru": (cudaRoundMode.cudaRoundPosInf, oracle.RU), "rd": (cudaRoundMode.cudaRoundMinInf, oracle.RD)}
RZ, RU = cudaRoundMode.cudaRoundZero, cudaRoundMode.cudaRoundPosInf


@pytest.fixture(scope="module")
def gold(golden_dir):
    return np.load(os.path.join(golden_dir, "value_types_reference.npz"))


def all_codes(repeat=37, extra=5):
    """Every code many times over, in an order that changes from copy to copy, with a
    ragged tail: long enough for the vector kernel, its last block and the scalar end."""
    rng = np.random.default_rng(5)
    return np.concatenate([rng.permutation(256) for _ in range(repeat)] + [np.arange(extra)]).astype(np.uint8)


def nan16(bits):
    return (bits & 0x7FFF) > 0x7F80


@pytest.mark.parametrize("fname", FORMATS)
@pytest.mark.parametrize("iname", INT_NAMES)
def test_value_to_integers(gold, fname, iname):
    codes = all_codes()
    got = cast(codes, fname, iname, rounding=RZ).copy_to_host()
    assert got.dtype == np.dtype(iname)
    assert np.array_equal(got, oracle.value_to(codes, FORMATS[fname], INTS[iname]))
    assert np.array_equal(got, gold[f"{fname}_to_{iname}"][codes])


@pytest.mark.parametrize("fname", FORMATS)
def test_value_to_floats_and_bool(gold, fname):
    codes = all_codes()
    fmt = FORMATS[fname]
    got = cast(codes, fname, "bool").copy_to_host()
    assert got.dtype == np.bool_ and np.array_equal(got.view(np.uint8), gold[f"{fname}_to_bool"][codes])
    want = oracle.value_to(codes, fmt, oracle.F64)
    got = cast(codes, fname, "f64").copy_to_host()
    assert np.array_equal(np.isnan(got), np.isnan(want)) and np.array_equal(got[~np.isnan(got)], want[~np.isnan(want)])
    want = oracle.value_to(codes, fmt, oracle.F16)
    got = cast(codes, fname, "f16").copy_to_host()
    assert got.dtype == np.float16
    assert np.array_equal(np.isnan(got), np.isnan(want))
    assert np.array_equal(got[~np.isnan(got)].view(np.uint16), want[~np.isnan(want)].view(np.uint16))
    assert np.array_equal(got[~np.isnan(got)].view(np.uint16), gold[f"{fname}_to_f16"][codes][~np.isnan(want)])
    want = oracle.value_to(codes, fmt, oracle.BF16)
    got = cast(codes, fname, "bf16").copy_to_host().view(np.uint16)
    assert np.array_equal(nan16(got), nan16(want)) and np.array_equal(got[~nan16(got)], want[~nan16(want)])


@pytest.mark.parametrize("fname", FORMATS)
@pytest.mark.parametrize("iname", INT_NAMES)
def test_value_from_integers(gold, fname, iname):
    x = integers(iname)
    rounding = RU if fname == "e8m0" else cudaRoundMode.cudaRoundNearest
    got = cast(x, iname, fname, rounding=rounding).copy_to_host()
    want = oracle.value_from(x, INTS[iname], FORMATS[fname])
    bad = np.nonzero(got != want)[0]
    assert bad.size == 0, (x[bad[:5]], got[bad[:5]], want[bad[:5]])
    assert np.array_equal(got, gold[f"{fname}_from_{iname}"])
    # a long array (vector path with many blocks) against the restatement
    big = np.random.default_rng(8).integers(np.iinfo(iname).min, np.iinfo(iname).max, 200003, dtype=iname,
                                            endpoint=True)
    if fname != "e8m0":   # the E8M0 restatement is a Python loop: the short array above covers it
        assert cast(big, iname, fname).copy_to_host().tobytes() == \
            oracle.value_from(big, INTS[iname], FORMATS[fname]).tobytes()


@pytest.mark.parametrize("fname", FORMATS)
def test_value_from_half(gold, fname):
    halves = np.arange(65536, dtype=np.uint16).view(np.float16)
    rounding = RU if fname == "e8m0" else cudaRoundMode.cudaRoundNearest
    got = cast(halves, "f16", fname, rounding=rounding).copy_to_host()
    finite = ~np.isnan(halves)
    assert np.array_equal(got[finite], gold[f"{fname}_from_f16"][finite])
    nan_code = 0xFF if fname == "e8m0" else 0x7F
    assert ((got[~finite] & 0x7F) == (nan_code & 0x7F)).all()
    if fname != "e8m0":
        for sat in (0, 1):
            got = cast(halves, "f16", fname, saturate=sat).copy_to_host()
            assert np.array_equal(got[finite], gold[f"{fname}_from_f16_sat{sat}"][finite])
    else:
        for sat in (0, 1):
            for mode, omode in ((RZ, oracle.RZ), (RU, oracle.RU)):
                got = cast(halves, "f16", "e8m0", saturate=sat, rounding=mode).copy_to_host()
                want = oracle.cast_ex(halves.astype(np.float32), oracle.F32, oracle.E8M0, sat, omode)
                assert np.array_equal(got, want)


@pytest.mark.parametrize("iname", [n for n in INT_NAMES if n not in ("int8", "uint8")])
@pytest.mark.parametrize("mode", MODES)
def test_integers_to_bf16(gold, iname, mode):
    x = integers(iname)
    got = cast(x, iname, "bf16", rounding=MODES[mode][0]).copy_to_host().view(np.uint16)
    want = oracle.int_to_bf16(x, INTS[iname], MODES[mode][1])
    bad = np.nonzero(got != want)[0]
    assert bad.size == 0, (x[bad[:5]], got[bad[:5]], want[bad[:5]])
    if mode == "rn":
        assert np.array_equal(got, gold[f"bf16_rn_from_{iname}"])
    fn = getattr(b16, f"{iname}_to_bfloat16_{mode}")
    assert np.asarray(fn(np.dtype(iname).type(257))).view(np.uint16) == (0x4381 if mode == "ru" else 0x4380)


@pytest.mark.parametrize("iname", INT_NAMES)
@pytest.mark.parametrize("mode", MODES)
def test_bf16_to_integers(gold, iname, mode):
    every = np.arange(65536, dtype=np.uint16)
    if iname in ("int8", "uint8") and mode != "rz":
        with pytest.raises(NotImplementedError):
            cast(every, "bf16", iname, rounding=MODES[mode][0])
        return
    got = cast(every, "bf16", iname, rounding=MODES[mode][0]).copy_to_host()
    want = oracle.bf16_to_int(every, INTS[iname], MODES[mode][1])
    bad = np.nonzero(got != want)[0]
    assert bad.size == 0, (every[bad[:5]], got[bad[:5]], want[bad[:5]])
    if mode == "rz":
        assert np.array_equal(got[bf16_patterns()], gold[f"bf16_to_{iname}_rz"])
    fn = getattr(b16, f"bfloat16_to_{iname}_{mode}")
    two_and_a_half = np.uint16(0x4020)
    assert fn(two_and_a_half) == {"rn": 2, "rz": 2, "rd": 2, "ru": 3}[mode]


def test_constructors_take_every_numeric_type():
    # numba_cuda/numba/cuda/tests/cudapy/test_fp8_bindings.py:62-160: 1.0 from every float
    # type, 2 (4 for E8M0) from every integer type, read back as float32
    import ml_dtypes
    for ctor, back, fval, ival in ((fp8_e4m3, fp8_e4m3_to, 1.0, 2), (fp8_e5m2, fp8_e5m2_to, 1.0, 2),
                                   (fp8_e8m0, fp8_e8m0_to, 2.0, 4)):
        for t in (np.float16, np.float32, np.float64, ml_dtypes.bfloat16):
            assert back(ctor(t(fval)), np.float32) == fval
        assert back(ctor(fval), np.float32) == fval                    # a Python float is a float64
        for name in INT_NAMES:
            assert back(ctor(np.dtype(name).type(ival)), np.float32) == float(ival)
        assert back(ctor(ival), np.float32) == float(ival)              # a Python int is an int64
    with pytest.raises(TypeError):
        fp8_e4m3(np.complex64(1))
    # a double is rounded once: 1 + 2^-4 + 2^-40 lies above the tie between 1.0 and 1.125
    tricky = 1.0 + 2.0 ** -4 + 2.0 ** -40
    assert fp8_e4m3(tricky) == 0x39 and fp8_e4m3(np.float32(tricky)) == 0x38


def test_conversion_operators_of_the_reference_tests():
    # test_fp8_bindings.py:186-330: to the float types, to unsigned and signed integers
    import ml_dtypes
    for ctor, back, val in ((fp8_e5m2, fp8_e5m2_to, 1.5), (fp8_e4m3, fp8_e4m3_to, 2.5), (fp8_e8m0, fp8_e8m0_to, 8.0)):
        v = ctor(np.float32(val))
        for t in (np.float16, np.float32, np.float64, ml_dtypes.bfloat16):
            assert float(back(v, t)) == val
    for ctor, back, val in ((fp8_e5m2, fp8_e5m2_to, 10.0), (fp8_e4m3, fp8_e4m3_to, 12.0), (fp8_e8m0, fp8_e8m0_to, 16.0)):
        v = ctor(np.float32(val))
        for t in (np.uint8, np.uint16, np.uint32, np.uint64):
            assert back(v, t) == int(val) and back(v, t).dtype == np.dtype(t)
    for ctor, back, pos, neg in ((fp8_e5m2, fp8_e5m2_to, 16.0, -8.0), (fp8_e4m3, fp8_e4m3_to, 20.0, -6.0),
                                 (fp8_e8m0, fp8_e8m0_to, 32.0, 16.0)):
        for t in (np.int8, np.int16, np.int32, np.int64):
            assert back(ctor(np.float32(pos)), t) == int(pos) and back(ctor(np.float32(neg)), t) == int(neg)
    for ctor, back in ((fp8_e5m2, fp8_e5m2_to), (fp8_e4m3, fp8_e4m3_to)):
        assert back(ctor(np.float32(0.0)), np.int64) == 0 and not back(ctor(np.float32(0.0)), bool)
        assert back(ctor(np.float32(np.nan)), np.int32) == 0
        assert back(ctor(np.float32(np.nan)), np.uint64) == np.uint64(1 << 63)
        assert back(ctor(np.float32(-3.0)), np.float32) == -3.0 and back(ctor(np.float32(-3.0)), np.int32) == -3
    assert fp8_e8m0_to(fp8_e8m0(np.float32(0.5)), bool)


def test_packed_types():
    rng = np.random.default_rng(12)
    x = (rng.standard_normal((1000, 4)) * 40).astype(np.float32)
    quads = fp8x4_e4m3(cuda.to_device(x)).copy_to_host()
    codes = oracle.cast(x, oracle.F32, oracle.E4M3, 1)
    assert quads.dtype == np.uint32 and quads.shape == (1000,)
    assert np.array_equal(quads, codes.view(np.uint32).reshape(1000))
    back = fp8x4_to(cuda.to_device(quads), "e4m3").copy_to_host()
    assert back.shape == (1000, 4) and np.array_equal(back, oracle.cast(codes, oracle.E4M3, oracle.F32))
    pairs = fp8x2_e4m3(cuda.to_device(x.reshape(2000, 2))).copy_to_host()
    assert pairs.dtype == np.uint16 and np.array_equal(pairs, codes.view(np.uint16).reshape(2000))
    R = oracle.ref_headers() if oracle.have_ref_headers() else None
    if R is not None:   # lane 0 in the low byte, as __nv_cvt_float2_to_fp8x2
        for i in range(0, 2000, 97):
            assert pairs[i] == R.ref_cvt_float2_to_fp8x2(float(x.reshape(-1)[2 * i]), float(x.reshape(-1)[2 * i + 1]), 1, 0)
    # a single pair / quadruple on the host gives a scalar
    assert fp8x2_e4m3(np.float32([1.0, -2.0])) == 0xC038
    assert fp8x4_e5m2(np.float64([1.0, 2.0, 4.0, -1.0])) == 0xBC44403C
    assert fp8x2_e8m0(np.float32([1.0, 3.0])) == ((129 << 8) | 127)
    halves = fp8x2_to(np.uint16(0xC038), "e4m3", np.float16)
    assert halves.dtype == np.float16 and halves.tolist() == [1.0, -2.0]
    d = x.astype(np.float64)
    assert np.array_equal(fp8x4_e5m2(cuda.to_device(d)).copy_to_host(),
                          oracle.cast_ex(d, oracle.F64, oracle.E5M2, 1).view(np.uint32).reshape(1000))


def test_unaligned_views_take_the_scalar_kernel():
    codes = all_codes()
    d = cuda.to_device(codes)
    for off in (1, 3):
        got = cast(d[off:], "e4m3", "int32", rounding=RZ).copy_to_host()
        assert np.array_equal(got, oracle.value_to(codes[off:], oracle.E4M3, oracle.I32))
    x = integers("int32")
    got = cast(cuda.to_device(x)[1:], "int32", "bf16").copy_to_host().view(np.uint16)
    assert np.array_equal(got, oracle.int_to_bf16(x[1:], oracle.I32, oracle.RN))


def test_modes_that_do_not_exist_are_refused():
    L = _lib.lib()
    x = cuda.to_device(np.zeros(64, np.int32))
    out = cuda.device_array(64, np.uint8)
    for sat, mode in ((0, _lib.ROUND_NEAREST), (1, _lib.ROUND_ZERO)):   # constructors saturate and round to nearest
        assert L.b2k_cast_ex(_lib.FMT_I32, _lib.FMT_E4M3, sat, mode, x._ptr, out._ptr, 64, None) == -2
    assert L.b2k_cast_ex(_lib.FMT_I32, _lib.FMT_E8M0, 1, _lib.ROUND_ZERO, x._ptr, out._ptr, 64, None) == -2
    assert L.b2k_cast_ex(_lib.FMT_E4M3, _lib.FMT_I32, 1, _lib.ROUND_NEAREST, out._ptr, x._ptr, 64, None) == -2
    assert L.b2k_cast_ex(_lib.FMT_I32, _lib.FMT_U32, 1, 0, x._ptr, x._ptr, 64, None) == -2
    assert L.b2k_cast_ex(_lib.FMT_I8, _lib.FMT_BF16, 1, 0, out._ptr, x._ptr, 64, None) == -2


def test_reference_bfloat16_integer_cases():
    """The cases of the reference's own tests (numba_cuda/numba/cuda/tests/cudapy/
    test_bfloat16.py:346-517): bit-cast round trip, 1.5 to every integer type in every
    mode, 789 from every integer type in every mode."""
    import ml_dtypes
    one_and_a_half = np.int16(0x3FC0)
    a = b16.int16_as_bfloat16(one_and_a_half)
    assert a.dtype == ml_dtypes.bfloat16 and float(a) == 1.5
    assert b16.bfloat16_as_int16(a) == one_and_a_half
    assert b16.bfloat16_as_uint16(b16.uint16_as_bfloat16(np.uint16(0x3FC0))) == 0x3FC0
    assert b16.bfloat16_to_int8_rz(a) == 1 and b16.bfloat16_to_uint8_rz(a) == 1
    for name in ("int16", "uint16", "int32", "uint32", "int64", "uint64"):
        got = [getattr(b16, f"bfloat16_to_{name}_{m}")(a) for m in ("rn", "rz", "rd", "ru")]
        assert [int(v) for v in got] == [2, 1, 1, 2] and all(v.dtype == np.dtype(name) for v in got)
        want = np.dtype(name).type(789).astype(ml_dtypes.bfloat16).view(np.int16)
        for m in ("rn", "rz", "rd", "ru"):
            bits = np.asarray(getattr(b16, f"{name}_to_bfloat16_{m}")(np.dtype(name).type(789))).view(np.int16)
            assert abs(int(bits) - int(want)) < 2, (name, m)
        # 789 = 0b1100010101 needs ten bits: 788 below, 792 above, 788 nearest
        exact = {"rn": 788.0, "rz": 788.0, "rd": 788.0, "ru": 792.0}
        for m, v in exact.items():
            assert float(getattr(b16, f"{name}_to_bfloat16_{m}")(np.dtype(name).type(789))) == v


def test_reference_fp8_nan_and_round_trip_cases():
    """numba_cuda/numba/cuda/tests/cudapy/test_fp8_bindings.py:162-177, :334-378: a NaN
    constructs a NaN in every fp8 type and converts to a NaN in float16 / float32 /
    float64; 4.0 survives the round trip through every type."""
    nan = np.float32(np.nan)
    for ctor, back in ((fp8_e5m2, fp8_e5m2_to), (fp8_e4m3, fp8_e4m3_to), (fp8_e8m0, fp8_e8m0_to)):
        code = ctor(nan)
        for t in (np.float16, np.float32, np.float64):
            assert np.isnan(back(code, t)), (ctor.__name__, t)
        assert back(ctor(np.float32(4.0)), np.float32) == 4.0
    assert fp8_e5m2(nan) & 0x7F > 0x7C and fp8_e4m3(nan) & 0x7F == 0x7F and fp8_e8m0(nan) == 0xFF
