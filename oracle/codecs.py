"""Bit-level codecs of the storage formats on the path (test infrastructure).

e4m3fn / e5m2 / e2m1 encode with IEEE round-to-nearest-even and saturation to
the largest finite value, which is what `static_cast<fp8>(clamped float)` does
in the reference (csrc/include/primus_turbo/float8.h:86-97, inputs are already
clamped by QuantOpBase::quant, device/quant_utils.cuh:33-40) and what the OCP
MX specification prescribes for the scaled converts used by the MX kernels
(csrc/kernels/quantization/quantization_mxfp8.cu:125-173,
quantization_mxfp4.cu:195-227).  ue8m0 is a bare biased exponent
(device/utils.cuh:124-126).
"""
from __future__ import annotations

import numpy as np

E4M3 = "e4m3"
E5M2 = "e5m2"
E2M1 = "e2m1"

# name -> (exponent bits, mantissa bits, bias, largest finite, NaN code)
_FMT = {
    E4M3: (4, 3, 7, 448.0, 0x7F),
    E5M2: (5, 2, 15, 57344.0, 0x7F),
    E2M1: (2, 1, 1, 6.0, 0x0),  # e2m1 has no NaN; NaN inputs are not produced on this path
}

# csrc/pytorch/quantization/quantization.cpp:23-37
FP8_MAX = {E4M3: 448.0, E5M2: 57344.0}
# csrc/include/primus_turbo/quantization.h:86-99 : (mantissa bits, target max pow2)
MX_PARAMS = {E4M3: (3, 8), E5M2: (2, 15), E2M1: (1, 2)}


def encode(x, fmt: str) -> np.ndarray:
    """float32 -> code (uint8; for e2m1 the low 4 bits). RNE, saturate to max finite."""
    ebits, mbits, bias, fmax, nan_code = _FMT[fmt]
    x = np.asarray(x, dtype=np.float32)
    sign = np.signbit(x).astype(np.uint8)
    a = np.abs(x).astype(np.float64)
    nan = np.isnan(a)
    a = np.where(nan, 0.0, a)
    a = np.minimum(a, fmax * 4.0)  # keep ldexp finite; still saturates below
    emin = 1 - bias
    _, e = np.frexp(a)
    fl = e - 1  # floor(log2(a)) for a > 0
    qexp = np.maximum(fl, emin) - mbits
    r = np.rint(np.ldexp(a, -qexp))  # ties to even, exact in float64
    val = np.minimum(np.ldexp(r, qexp), fmax)
    _, e2 = np.frexp(val)
    fl2 = e2 - 1
    sub = (val == 0.0) | (fl2 < emin)
    exp_field = np.where(sub, 0, fl2 + bias).astype(np.int64)
    mant_sub = np.ldexp(val, -(emin - mbits))
    mant_nrm = (np.ldexp(val, -fl2) - 1.0) * (1 << mbits)
    mant = np.where(sub, mant_sub, mant_nrm).astype(np.int64)
    code = (exp_field << mbits) | mant
    code = code | (sign.astype(np.int64) << (ebits + mbits))
    if fmt != E2M1:
        code = np.where(nan, nan_code | (sign.astype(np.int64) << 7 if fmt == E4M3 else 0), code)
    return code.astype(np.uint8)


def _decode_table(fmt: str) -> np.ndarray:
    ebits, mbits, bias, _, _ = _FMT[fmt]
    n = 1 << (1 + ebits + mbits)
    t = np.zeros(n, dtype=np.float32)
    for c in range(n):
        s = -1.0 if (c >> (ebits + mbits)) & 1 else 1.0
        ef = (c >> mbits) & ((1 << ebits) - 1)
        mf = c & ((1 << mbits) - 1)
        if ef == 0:
            v = mf * 2.0 ** (1 - bias - mbits)
        else:
            v = (1.0 + mf / (1 << mbits)) * 2.0 ** (ef - bias)
        if fmt == E4M3 and ef == 15 and mf == 7:
            v = float("nan")
        if fmt == E5M2 and ef == 31:
            v = float("inf") if mf == 0 else float("nan")
        t[c] = s * v
    return t


_TABLES = {f: _decode_table(f) for f in _FMT}


def decode(code, fmt: str) -> np.ndarray:
    """code (uint8) -> float32."""
    code = np.asarray(code, dtype=np.uint8)
    if fmt == E2M1:
        code = code & 0xF
    return _TABLES[fmt][code]


def pack_e2m1(codes: np.ndarray) -> np.ndarray:
    """[..., 2k] 4-bit codes -> [..., k] bytes; element 2j in the low nibble
    (quantization_mxfp4.cu:198-213, dequantization_mxfp4.cu:26-27)."""
    codes = np.asarray(codes, dtype=np.uint8)
    return (codes[..., 0::2] & 0xF) | ((codes[..., 1::2] & 0xF) << 4)


def unpack_e2m1(packed: np.ndarray) -> np.ndarray:
    packed = np.asarray(packed, dtype=np.uint8)
    out = np.empty(packed.shape[:-1] + (packed.shape[-1] * 2,), dtype=np.uint8)
    out[..., 0::2] = packed & 0xF
    out[..., 1::2] = packed >> 4
    return out


def e8m0_to_f32(byte) -> np.ndarray:
    """2^(byte-127) built as (byte << 23) reinterpret; byte 0 gives 0.0f exactly as the
    quantizer's `r_scale_native` (quantization_mxfp8.cu:103)."""
    b = np.asarray(byte, dtype=np.uint32)
    return (b << np.uint32(23)).view(np.float32)


def e8m0_decode(byte) -> np.ndarray:
    """Dequantize-side value of a ue8m0 byte: (byte << 23) reinterpreted as float32 (device/utils.cuh:124-126), i.e.
    2^(byte - 127) for bytes 1..254, 0.0 for byte 0 and +inf for byte 255.  Pinned for all 256 bytes by
    tests/golden/mx.npz (the reference's e8m0_to_scale compiled on the host)."""
    return e8m0_to_f32(byte)


def mx_scale_from_amax(amax, fmt: str):
    """ue8m0 byte and native scale from a block amax
    (quantization_mxfp8.cu:68-105, quantization_mxfp4.cu:149-181)."""
    mbits, target = MX_PARAMS[fmt]
    bits = np.asarray(amax, dtype=np.float32).view(np.uint32).astype(np.int64)
    val_to_add = 1 << (23 - mbits - 1)
    e = (((bits + val_to_add) >> 23) & 0x1FF) - 127 - target
    e = np.clip(e, -127, 128)
    byte = (e + 127).astype(np.uint8)
    return byte, e8m0_to_f32(byte)


def bf16_round(x) -> np.ndarray:
    """float32 -> nearest bf16 (RNE), returned as float32."""
    u = np.asarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    lsb = (u >> 16) & 1
    u = (u + 0x7FFF + lsb) & 0xFFFF0000
    return u.astype(np.uint32).view(np.float32)
