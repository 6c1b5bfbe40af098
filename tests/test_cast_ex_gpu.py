"""The remaining conversion intrinsics as bulk casts (directed rounding to bf16,
float64 -> bf16, the E8M0 scale type, float16) on the GPU against the
reference's vendored headers (fixtures) and the C restatement."""
import os

import numpy as np
import pytest

import oracle
import numba_cuda_b200 as cuda
from numba_cuda_b200 import _lib
from numba_cuda_b200.casts import (cast, cudaRoundMode, cvt_bfloat16raw_to_e8m0, cvt_e8m0_to_bf16raw,
                                   cvt_float_to_e8m0, float32_to_bfloat16_rd, float32_to_bfloat16_ru,
                                   float32_to_bfloat16_rz, float64_to_bfloat16, fp8_e8m0_to_float32,
                                   saturation_t)

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
        cast(np.zeros(8, dtype=np.float64), "f64", "e4m3")
    with pytest.raises(NotImplementedError):
        cast(np.zeros(8, dtype=np.float32), "f32", "e4m3", rounding=RZ)
    L = _lib.lib()
    assert L.b2k_cast_ex(_lib.FMT_F32, _lib.FMT_BF16, 1, 9, 1024, 2048, 8, None) == _lib.ERR_INVALID_ARG
