"""The CPU restatement of the conversions with an integer side (oracle.value_to /
value_from / int_to_bf16 / bf16_to_int) against outputs of the reference's own
vendored headers: the committed fixture always, the compiled headers when present."""
import os

import numpy as np
import pytest

import oracle
from value_type_inputs import INT_NAMES, bf16_patterns, integers

FORMATS = {"e4m3": oracle.E4M3, "e5m2": oracle.E5M2, "e8m0": oracle.E8M0}
FLOATS = {"f16": oracle.F16, "bf16": oracle.BF16, "f32": oracle.F32, "f64": oracle.F64}
INTS = {name: getattr(oracle, "I" + name[3:] if name.startswith("int") else "U" + name[4:]) for name in INT_NAMES}
CODES = np.arange(256, dtype=np.uint8)


@pytest.fixture(scope="module")
def gold(golden_dir):
    return np.load(os.path.join(golden_dir, "value_types_reference.npz"))


def same_floats(got, want, bits16=None):
    """Equal where the reference has a number; a NaN wherever it has a NaN."""
    if bits16 == "bf16":
        gnan, wnan = (got & 0x7FFF) > 0x7F80, (want & 0x7FFF) > 0x7F80
    else:
        gnan, wnan = np.isnan(got), np.isnan(want)
    return np.array_equal(gnan, wnan) and np.array_equal(got[~gnan], want[~wnan])


@pytest.mark.parametrize("fname", FORMATS)
def test_conversion_operators_match_reference(gold, fname):
    fmt = FORMATS[fname]
    for tname, dst in FLOATS.items():
        want = gold[f"{fname}_to_{tname}"]
        if tname == "f16":
            want = want.view(np.float16)
        assert same_floats(oracle.value_to(CODES, fmt, dst), want, tname), tname
    for iname, dst in INTS.items():
        assert np.array_equal(oracle.value_to(CODES, fmt, dst), gold[f"{fname}_to_{iname}"]), iname
    assert np.array_equal(oracle.value_to(CODES, fmt, oracle.BOOL), gold[f"{fname}_to_bool"])


def test_conversion_known_answers():
    # the cases of the reference's tests: values that convert exactly, negative and zero, NaN
    e4, e5, e8 = oracle.E4M3, oracle.E5M2, oracle.E8M0
    assert oracle.value_to(oracle.cast(np.float32([12.0, -6.0, 20.0, 0.0]), oracle.F32, e4), e4, oracle.I32).tolist() == \
        [12, -6, 20, 0]
    assert oracle.value_to(oracle.cast(np.float32([10.0, -8.0, 16.0]), oracle.F32, e5), e5, oracle.I64).tolist() == [10, -8, 16]
    assert oracle.value_to(np.uint8([127 + 4, 127 + 5]), e8, oracle.U16).tolist() == [16, 32]
    assert oracle.value_to(np.uint8([0x7F, 0xFF]), e4, oracle.I32).tolist() == [0, 0]          # NaN
    assert oracle.value_to(np.uint8([0x7F]), e4, oracle.U64)[0] == 1 << 63
    assert oracle.value_to(np.uint8([0x7C, 0xFC]), e5, oracle.I16).tolist() == [32767, -32768]  # infinities
    assert oracle.value_to(np.uint8([0x00, 0x80, 0x01, 0x7F]), e4, oracle.BOOL).tolist() == [0, 0, 1, 1]
    assert oracle.value_to(np.uint8([0x00]), e8, oracle.BOOL).tolist() == [1]


@pytest.mark.parametrize("fname", FORMATS)
def test_constructors_from_integers_match_reference(gold, fname):
    fmt = FORMATS[fname]
    for iname, src in INTS.items():
        x = integers(iname)
        got = oracle.value_from(x, src, fmt)
        want = gold[f"{fname}_from_{iname}"]
        bad = np.nonzero(got != want)[0]
        assert bad.size == 0, (iname, x[bad[:5]], got[bad[:5]], want[bad[:5]])


@pytest.mark.parametrize("fname", FORMATS)
def test_constructors_from_half_match_reference(gold, fname):
    halves = np.arange(65536, dtype=np.uint16).view(np.float16)
    got = oracle.value_from(halves, oracle.F16, FORMATS[fname])
    assert np.array_equal(got, gold[f"{fname}_from_f16"])
    if fname != "e8m0":
        finite = ~np.isnan(halves)
        for sat in (0, 1):
            via_float = oracle.cast(halves.astype(np.float32), oracle.F32, FORMATS[fname], sat)
            assert np.array_equal(via_float[finite], gold[f"{fname}_from_f16_sat{sat}"][finite])


def test_constructor_known_answers():
    # 1.0 / 2 from every source type, as the reference's constructor tests
    for fmt, one, two in ((oracle.E4M3, 0x38, 0x40), (oracle.E5M2, 0x3C, 0x40)):
        for src, arr in ((oracle.F16, np.float16([1.0])), (oracle.F32, np.float32([1.0])), (oracle.F64, np.float64([1.0]))):
            assert oracle.value_from(arr, src, fmt)[0] == one
        for iname, src in INTS.items():
            assert oracle.value_from(np.array([2], dtype=iname), src, fmt)[0] == two
    for iname, src in INTS.items():
        assert oracle.value_from(np.array([4, 5, 1, 0], dtype=iname), src, oracle.E8M0).tolist()[:3] == [129, 130, 127]


def test_bf16_to_integers_toward_zero_matches_reference(gold):
    pats = bf16_patterns()
    for iname, dst in INTS.items():
        got = oracle.bf16_to_int(pats, dst, oracle.RZ)
        want = gold[f"bf16_to_{iname}_rz"]
        bad = np.nonzero(got != want)[0]
        assert bad.size == 0, (iname, pats[bad[:5]], got[bad[:5]], want[bad[:5]])


def test_integers_to_bf16_nearest_matches_reference(gold):
    for iname, src in INTS.items():
        if iname in ("int8", "uint8"):
            continue
        x = integers(iname)
        got = oracle.int_to_bf16(x, src, oracle.RN)
        want = gold[f"bf16_rn_from_{iname}"]
        bad = np.nonzero(got != want)[0]
        assert bad.size == 0, (iname, x[bad[:5]], got[bad[:5]], want[bad[:5]])


def test_directed_modes_bracket_the_value():
    """The modes without a host path in the reference's header are pinned by what
    defines them: toward -inf <= value <= toward +inf, both next to each other in
    bfloat16, toward zero the one of smaller magnitude, nearest one of the two."""
    def value(bits):
        with np.errstate(invalid="ignore"):
            return (bits.astype(np.uint32) << 16).view(np.float32).astype(np.float64)
    for iname in ("int16", "int32", "int64", "uint16", "uint32", "uint64"):
        x = integers(iname, n=1024)
        down, up = oracle.int_to_bf16(x, INTS[iname], oracle.RD), oracle.int_to_bf16(x, INTS[iname], oracle.RU)
        zero, near = oracle.int_to_bf16(x, INTS[iname], oracle.RZ), oracle.int_to_bf16(x, INTS[iname], oracle.RN)
        for i, v in enumerate(int(t) for t in x):
            lo, hi = value(down[i:i + 1])[0], value(up[i:i + 1])[0]
            assert int(lo) <= v <= int(hi)
            assert zero[i] == (down[i] if v >= 0 else up[i])
            assert near[i] in (down[i], up[i])
            if int(lo) != int(hi):   # neighbours in bfloat16: one step apart in the bit pattern
                assert abs(int(down[i] & 0x7FFF) - int(up[i] & 0x7FFF)) == 1
    pats = bf16_patterns()
    vals = value(pats)
    finite = np.isfinite(vals) & (np.abs(vals) < 2.0 ** 31)
    for mode, fn in ((oracle.RN, np.rint), (oracle.RU, np.ceil), (oracle.RD, np.floor)):
        got = oracle.bf16_to_int(pats, oracle.I64, mode)
        assert np.array_equal(got[finite], fn(vals[finite]).astype(np.int64))


@pytest.mark.skipif(not oracle.have_ref_headers(), reason="reference-header checker not built")
def test_fixture_is_what_the_compiled_headers_give(gold):
    for fname, fmt in FORMATS.items():
        for iname, dst in INTS.items():
            assert np.array_equal(oracle.ref_value_to(CODES, fmt, dst), gold[f"{fname}_to_{iname}"])
            assert np.array_equal(oracle.ref_value_from(integers(iname), dst, fmt), gold[f"{fname}_from_{iname}"])
