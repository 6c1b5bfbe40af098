"""The CPU oracle against fixtures produced by executing the reference
(tests/golden/make_golden.py) and against the known-answer values of the
reference's own tests.  No GPU."""
import os

import numpy as np
import pytest

import oracle


def pairs(st):
    return np.stack([st["s0"], st["s1"]], axis=1)


@pytest.fixture(scope="module")
def rng_gold(golden_dir):
    return np.load(os.path.join(golden_dir, "rng_reference.npz"))


@pytest.fixture(scope="module")
def cast_gold(golden_dir):
    return np.load(os.path.join(golden_dir, "cast_reference.npz"))


@pytest.fixture(scope="module")
def reduce_gold(golden_dir):
    return np.load(os.path.join(golden_dir, "reduce_reference.npz"))


def test_states_match_reference(rng_gold):
    assert (pairs(oracle.init_states(64, 42, 0)) == rng_gold["states_seed42_n64"]).all()
    assert (pairs(oracle.init_states(4, 1, 0)) == rng_gold["states_seed1_n4"]).all()
    assert (pairs(oracle.init_states(8, 1, 2)) == rng_gold["states_seed1_start2_n8"]).all()
    assert (pairs(oracle.init_states(4, 7, 1000)) == rng_gold["states_seed7_start1000_n4"]).all()


def test_known_state_values():
    # values obtained by running the reference's CPU-jitted init
    st = oracle.init_states(2, 42, 0)
    assert int(st[0]["s0"]) == 0xBDD732262FEB6E95 == int(st[0]["s1"])
    assert (int(st[1]["s0"]), int(st[1]["s1"])) == (313611670190079035, 410834281257317300)


def test_long_chain_matches_reference(rng_gold):
    big = oracle.init_states(1 << 20, 42, 0)
    assert (pairs(big[rng_gold["big_idx"]]) == rng_gold["big_states_seed42"]).all()
    assert (pairs(big[:: int(rng_gold["big_stride"])]) == rng_gold["big_states_seed42_strided"]).all()


def test_subsequence_identity():
    # tests/cudapy/test_random.py:62-72
    s1 = oracle.init_states(10, 1, 0)
    s2 = oracle.init_states(10, 1, 3)
    assert (pairs(s1)[3:] == pairs(s2)[:-3]).all()


@pytest.mark.parametrize("dist,dtype,key,count", [
    ("uniform", np.float32, "uniform_f32", 64), ("uniform", np.float64, "uniform_f64", 64),
    ("normal", np.float32, "normal_f32_hostlibm", 32), ("normal", np.float64, "normal_f64_hostlibm", 32)])
def test_draws_match_reference_cpu_path(rng_gold, dist, dtype, key, count):
    st = oracle.init_states(4, 42, 0)
    got = oracle.fill(st, dist, dtype, count)
    want = rng_gold[key]
    if dist == "uniform":
        assert got.tobytes() == want.tobytes()
    else:  # host libm on both sides, but allow an ulp in case libm versions differ
        np.testing.assert_allclose(got, want, rtol=4 * np.finfo(dtype).eps)
    end_key = key.replace("_hostlibm", "") + "_end"
    assert (pairs(st) == rng_gold[end_key]).all()


def test_config4_sequence(rng_gold):
    st = oracle.init_states(8, 42, 0)
    u = oracle.fill(st, "uniform", np.float32, 64)
    z = oracle.fill(st, "normal", np.float64, 16)
    assert u.tobytes() == rng_gold["c4_u"].tobytes()
    np.testing.assert_allclose(z, rng_gold["c4_z_hostlibm"], rtol=1e-15)
    assert (pairs(st) == rng_gold["c4_end"]).all()


def test_uniform_moments():
    # tests/cudapy/test_random.py:82-97
    st = oracle.init_states(64, 1, 0)
    u = oracle.fill(st, "uniform", np.float32, 32).ravel()
    assert abs(u.min()) < 1e-3 and abs(u.max() - 1.0) < 1e-3
    assert abs(u.mean() - 0.5) < 1.5e-2 and abs(u.std() - 1 / (2 * 3 ** 0.5)) < 6e-3


@pytest.mark.parametrize("name,dst", [("e4m3", oracle.E4M3), ("e5m2", oracle.E5M2)])
def test_fp8_matches_reference_headers(cast_gold, name, dst):
    x = cast_gold["f32_bits"].view(np.float32)
    assert (oracle.cast(x, oracle.F32, dst, 1) == cast_gold[f"{name}_satfinite"]).all()
    assert (oracle.cast(x, oracle.F32, dst, 0) == cast_gold[f"{name}_nosat"]).all()
    codes = np.arange(256, dtype=np.uint8)
    assert (oracle.cast(codes, dst, oracle.F32).view(np.uint32) == cast_gold[f"{name}_decode_f32_bits"]).all()
    half = np.array([oracle.lib().oracle_fp8_to_f16bits(int(c), dst - 2) for c in codes], dtype=np.uint16)
    assert (half == cast_gold[f"{name}_decode_half_bits"]).all()


def test_fp8_known_answers():
    # tests/cudapy/test_fp8_bindings.py:388-419 (1e20) and :88-128 (exact small values)
    L = oracle.lib()
    assert L.oracle_f32_to_fp8(1e20, 0, 1) == 0x7C and L.oracle_f32_to_fp8(1e20, 1, 1) == 0x7B
    assert L.oracle_f32_to_fp8(1e20, 0, 0) == 0x7F and L.oracle_f32_to_fp8(1e20, 1, 0) == 0x7E
    assert L.oracle_f64_to_fp8(1e300, 0, 1) == 0x7C and L.oracle_f64_to_fp8(1e300, 1, 0) == 0x7E
    for v in (1.0, 2.0, 4.0, -1.0, 0.5, 448.0, -448.0):
        for interp in (0, 1):
            assert L.oracle_fp8_to_f32(L.oracle_f32_to_fp8(v, 1, interp), interp) == v
    assert L.oracle_f32_to_fp8(float("nan"), 1, 0) == 0x7F
    assert np.isnan(L.oracle_fp8_to_f32(0x7F, 0)) and np.isnan(L.oracle_fp8_to_f32(0x7E, 1))
    # spot values checked against the vendored headers
    for v, code in ((448.0, 0x7E), (464.0, 0x7E), (465.0, 0x7E), (1e6, 0x7E), (float("inf"), 0x7E),
                    (float("-inf"), 0xFE), (2.0 ** -10, 0x00), (0.017, 0x09)):
        assert L.oracle_f32_to_fp8(v, 1, 0) == code, v


def test_bf16_matches_reference_headers(cast_gold):
    x = cast_gold["f32_bits"].view(np.float32)
    assert (oracle.cast(x, oracle.F32, oracle.BF16) == cast_gold["bf16_rn"]).all()
    # tests/cudapy/test_bfloat16.py:518-529: 1.5 is exact
    assert oracle.lib().oracle_bf16_to_f32(oracle.lib().oracle_f32_to_bf16(1.5)) == 1.5
    assert oracle.lib().oracle_f32_to_bf16(float("nan")) == 0x7FFF


def test_bf16_agrees_with_ml_dtypes_on_finite():
    ml_dtypes = pytest.importorskip("ml_dtypes")
    x = np.random.default_rng(2).standard_normal(1 << 16, dtype=np.float32)
    assert (oracle.cast(x, oracle.F32, oracle.BF16) == x.astype(ml_dtypes.bfloat16).view(np.uint16)).all()


@pytest.mark.skipif(not oracle.have_ref_headers(), reason="reference-header checker not built")
def test_restatement_equals_reference_headers_on_random_bits():
    bits = np.random.default_rng(11).integers(0, 2 ** 32, size=1 << 18, dtype=np.uint32)
    x = bits.view(np.float32)
    for dst in (oracle.E4M3, oracle.E5M2):
        for sat in (0, 1):
            assert (oracle.cast(x, oracle.F32, dst, sat) == oracle.ref_cast(x, oracle.F32, dst, sat)).all()
    assert (oracle.cast(x, oracle.F32, oracle.BF16) == oracle.ref_cast(x, oracle.F32, oracle.BF16)).all()
    h = np.arange(1 << 16, dtype=np.uint16)
    assert oracle.cast(h, oracle.BF16, oracle.F32).tobytes() == oracle.ref_cast(h, oracle.BF16, oracle.F32).tobytes()


def test_reduce_matches_simulator(reduce_gold):
    x = np.random.default_rng(0).random(1 << 20)
    assert oracle.fold(x, "add", 0) == reduce_gold["c1_sum"]
    y = np.random.default_rng(1).integers(-2 ** 31, 2 ** 31, size=int(reduce_gold["c2_prefix_len"]), dtype=np.int32)
    assert oracle.fold(y, "max", 0) == reduce_gold["c2_prefix_max"]
    A = np.arange(34567, dtype=np.float64) + 1
    assert oracle.fold(A, "add", 0) == reduce_gold["sum_arange_34567"] == A.sum()
    assert oracle.fold(np.arange(64, dtype=np.float64) + 1, "mul", 1) == reduce_gold["prod_64_init1"]
    assert oracle.fold(reduce_gold["max_input"], "max", 0) == reduce_gold["max_3717_init0"]
    assert oracle.fold(np.arange(10, dtype=np.float64) + 1, "add", 3) == reduce_gold["sum_10_init3"]
    assert oracle.py_fold(lambda a, b: a + b, [1, 2, 3], 3) == 9


def test_transpose_restatement():
    rng = np.random.default_rng(4)
    a = rng.integers(0, 255, size=(7, 12)).astype(np.int64)
    assert (oracle.transpose2d(a) == a.T).all()
    v = a[::2, ::2]
    assert (oracle.transpose2d(v) == v.T).all()
    rec = np.zeros((3, 5), dtype=np.dtype([("i", np.int32), ("j", np.float32, (3, 2))], align=True))
    rec["i"] = rng.integers(0, 100, size=(3, 5))
    assert (oracle.transpose2d(rec) == rec.T).all()


def test_directed_rounding_f64_and_e8m0_match_reference_headers(cast_gold):
    x = cast_gold["f32_bits"].view(np.float32)
    for mode, tag in ((oracle.RZ, "rz"), (oracle.RU, "ru"), (oracle.RD, "rd")):
        assert (oracle.cast_ex(x, oracle.F32, oracle.BF16, mode=mode) == cast_gold[f"bf16_{tag}"]).all(), tag
    h = np.arange(65536, dtype=np.uint16)
    for sat, stag in ((0, "nosat"), (1, "satfinite")):
        for mode, mtag in ((oracle.RZ, "rz"), (oracle.RU, "rp")):
            assert (oracle.cast_ex(x, oracle.F32, oracle.E8M0, sat, mode) == cast_gold[f"e8m0_from_f32_{stag}_{mtag}"]).all()
            assert (oracle.cast_ex(h, oracle.BF16, oracle.E8M0, sat, mode) == cast_gold[f"e8m0_from_bf16_{stag}_{mtag}"]).all()
    assert (oracle.cast_ex(np.arange(256, dtype=np.uint8), oracle.E8M0, oracle.BF16) == cast_gold["e8m0_to_bf16"]).all()
    assert (oracle.cast_ex(cast_gold["f64_inputs"], oracle.F64, oracle.BF16) == cast_gold["bf16_from_f64"]).all()
    # known answers of tests/cudapy/test_fp8_bindings.py:449-560
    L = oracle.lib()
    assert L.oracle_e8m0_to_bf16(127) == 0x3F80
    over = float(np.nextafter(np.float32(2.0 ** 127), np.float32(np.inf)))
    assert L.oracle_f32_to_e8m0(over, 0, oracle.RU) == 0xFF and L.oracle_f32_to_e8m0(over, 1, oracle.RU) == 0xFE
    half = L.oracle_e8m0_to_bf16(126)
    assert L.oracle_bf16_to_e8m0(half, 0, oracle.RZ) == 126 and L.oracle_bf16_to_e8m0(half, 0, oracle.RU) == 126


@pytest.mark.skipif(not oracle.have_ref_headers(), reason="reference-header checker not built")
def test_double_and_bf16raw_sources_match_reference_headers():
    """cvt_double_to_fp8, cvt_bfloat16raw_to_fp8, cvt_double_to_e8m0: restatement vs the
    vendored headers, plus the known answers of tests/cudapy/test_fp8_bindings.py:421-447,
    :463-496, :521-539."""
    rng = np.random.default_rng(12)
    x = np.concatenate([rng.standard_normal(1 << 17) * np.exp2(rng.uniform(-30, 30, 1 << 17)),
                        rng.integers(0, 2 ** 64, size=1 << 17, dtype=np.uint64).view(np.float64)])
    h = np.arange(1 << 16, dtype=np.uint16)
    for dst in (oracle.E4M3, oracle.E5M2):
        for sat in (0, 1):
            assert oracle.cast_ex(x, oracle.F64, dst, sat).tobytes() == oracle.ref_cast(x, oracle.F64, dst, sat).tobytes()
            assert oracle.cast_ex(h, oracle.BF16, dst, sat).tobytes() == oracle.ref_cast(h, oracle.BF16, dst, sat).tobytes()
    wide = np.concatenate([x, rng.standard_normal(1 << 16) * np.exp2(rng.uniform(-140, 140, 1 << 16))])
    for sat in (0, 1):
        for mode in (oracle.RZ, oracle.RU):
            assert oracle.cast_ex(wide, oracle.F64, oracle.E8M0, sat, mode).tobytes() == \
                oracle.ref_cast(wide, oracle.F64, oracle.E8M0, sat, mode=mode).tobytes()
    L = oracle.lib()
    assert [L.oracle_f64_to_fp8(1e300, s, i) for s, i in ((0, 1), (1, 1), (0, 0), (1, 0))] == [0x7C, 0x7B, 0x7F, 0x7E]
    raw = L.oracle_e8m0_to_bf16(254)
    assert [L.oracle_bf16_to_fp8(raw, s, i) for s, i in ((0, 1), (1, 1), (0, 0), (1, 0))] == [0x7C, 0x7B, 0x7F, 0x7E]
    over = float(np.nextafter(np.float64(2.0 ** 127), np.float64(np.inf)))
    assert L.oracle_f64_to_e8m0(over, 0, oracle.RU) == 0xFF and L.oracle_f64_to_e8m0(over, 1, oracle.RU) == 0xFE
