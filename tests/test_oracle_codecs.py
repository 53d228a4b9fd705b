"""Codec checks of the CPU oracle: torch's CPU fp8 casts as an independent opinion on
round-to-nearest-even, the e2m1 value grid, ue8m0 scale selection, and the MX round-trip
tolerances the reference's own tests use (tests/pytorch/ops/test_quantization.py:340-484,551-687)."""
import numpy as np
import pytest
import torch

from oracle import codecs as oc
from oracle import quant as oq


def _all_bf16():
    bits = np.arange(1 << 16, dtype=np.uint32) << 16
    v = bits.view(np.float32)
    return v[np.isfinite(v)]


@pytest.mark.parametrize("fmt,tdt", [("e4m3", torch.float8_e4m3fn), ("e5m2", torch.float8_e5m2)])
def test_fp8_encode_matches_torch_cpu_cast(fmt, tdt):
    v = _all_bf16()
    rng = np.random.default_rng(0)
    extra = (rng.standard_normal(200000) * rng.choice([1e-3, 1.0, 100.0], 200000)).astype(np.float32)
    v = np.concatenate([v, extra])
    v = np.clip(v, -oc.FP8_MAX[fmt], oc.FP8_MAX[fmt])  # the path always clamps before the cast
    want = torch.from_numpy(v).to(tdt).view(torch.uint8).numpy()
    got = oc.encode(v, fmt)
    assert np.array_equal(got, want)
    # decode is the exact inverse on the codes produced
    back = torch.from_numpy(want).view(tdt).to(torch.float32).numpy()
    assert np.array_equal(oc.decode(got, fmt), back)


def test_e2m1_grid_and_ties():
    grid = [0, 0.5, 1, 1.5, 2, 3, 4, 6]
    assert np.array_equal(oc.decode(np.arange(8, dtype=np.uint8), "e2m1"), np.array(grid, np.float32))
    # ties go to the even code; beyond 6 saturates
    x = np.array([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 7.0, 100.0, -0.25, -5.0], np.float32)
    want = np.array([0, 1.0, 1.0, 2.0, 2.0, 4.0, 4.0, 6.0, 6.0, -0.0, -4.0], np.float32)
    assert np.array_equal(oc.decode(oc.encode(x, "e2m1"), "e2m1"), want)
    c = np.arange(16, dtype=np.uint8).reshape(1, 16)
    assert np.array_equal(oc.unpack_e2m1(oc.pack_e2m1(c)), c)
    assert oc.pack_e2m1(np.array([[1, 2]], np.uint8))[0, 0] == 0x21  # element 0 in the low nibble


def test_mx_scale_rule():
    # amax whose top mantissa bits round up moves to the next exponent (quantization_mxfp8.cu:85-104)
    b, s = oc.mx_scale_from_amax(np.array([448.0, 1.0, 0.0, 1.90625, 1.9375], np.float32), "e4m3")
    assert list(b) == [127, 127 - 8, 0, 127 - 8, 127 - 7]
    assert s[2] == 0.0 and s[0] == 1.0
    b, _ = oc.mx_scale_from_amax(np.array([6.0, 7.0, 3.0], np.float32), "e2m1")
    assert list(b) == [127, 128, 126]


@pytest.mark.parametrize("fmt,tol", [("e4m3", 1e-1), ("e5m2", 1e-1), ("e2m1", 0.5)])
@pytest.mark.parametrize("axis", [0, 1])
@pytest.mark.parametrize("use_2d", [False, True])
def test_mx_round_trip(fmt, tol, axis, use_2d):
    rng = np.random.default_rng(3)
    M, N = 200, 96
    x = oc.bf16_round(rng.standard_normal((M, N)).astype(np.float32))
    q, s = oq.quantize_mx(x, fmt, axis, use_2d)
    d = oq.dequantize_mx(q, s, fmt)
    xp = np.zeros((256, 128), np.float32)
    xp[:M, :N] = x
    ref = xp[:M] if axis == 1 else xp[:, :N].T
    assert d.shape == ref.shape
    assert np.allclose(d, ref, rtol=tol, atol=tol)
    assert s.shape == (ref.shape[0], ref.shape[1] // 32)


def test_rht16_is_orthonormal_hadamard():
    rng = np.random.default_rng(1)
    x = rng.standard_normal((3, 32)).astype(np.float32)
    y = oq._rht16(x)
    assert np.allclose(np.sum(y * y, axis=1), np.sum(x * x, axis=1), rtol=1e-5)
    assert np.allclose(oq._rht16(y), x, atol=1e-5)  # H16/4 is an involution
