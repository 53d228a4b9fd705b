"""CPU restatement of the reference quantize / dequantize kernels (test infrastructure).

Inputs are float32 arrays holding the exact upcast of the bf16 / fp16 / fp32
source (bf16 -> fp32 is a 16-bit shift, device/utils.cuh:72-78).  All arithmetic
is done in float32 in the order the kernels use.  Outputs are raw bytes
(uint8), float32 scales, or ue8m0 bytes (uint8).
"""
from __future__ import annotations

import numpy as np

from .codecs import (E2M1, E4M3, E5M2, FP8_MAX, decode, e8m0_decode, encode,
                     mx_scale_from_amax, pack_e2m1, unpack_e2m1)

F32 = np.float32


def _amax(a: np.ndarray, axis=None, keepdims=False):
    """max |a| as the kernels take it: fmaxf(fabsf(x), fabsf(y)) (device/reduce.cuh:119-125, quantization_mxfp8.cu amax
    loops), which returns the other operand when one is NaN -- a NaN element takes no part in the maximum."""
    a = np.abs(a)
    if axis is None:
        return np.fmax.reduce(a.reshape(-1), initial=F32(0)) if a.size else F32(0)
    axes = (axis,) if isinstance(axis, int) else tuple(sorted((ax % a.ndim for ax in axis), reverse=True))
    out = a
    for ax in axes:
        out = np.fmax.reduce(out, axis=ax, keepdims=True, initial=F32(0))
    if not keepdims:
        out = np.squeeze(out, axis=tuple(sorted(ax % a.ndim for ax in axes)))
    return out


def _ceil_to(x: int, a: int) -> int:
    return (x + a - 1) // a * a


def _quant_clamp_encode(x: np.ndarray, scale, fmt: str) -> np.ndarray:
    """q = fp8_rne(fmax(fmin(x*scale, qmax), -qmax))   (device/quant_utils.cuh:33-40)."""
    qmax = F32(FP8_MAX[fmt])
    v = (x.astype(F32) * np.asarray(scale, dtype=F32)).astype(F32)
    v = np.fmax(np.fmin(v, qmax), -qmax)
    return encode(v, fmt)


def _scale_from_amax(amax, fmt: str, eps: float):
    """scale = qmax / fmax(amax, eps); scale_inv = 1.0f / scale
    (device/quant_utils.cuh:62-74; blockwise eps 1e-4: quantization_blockwise.cu:142,162,302)."""
    amax = np.fmax(np.asarray(amax, dtype=F32), F32(eps))
    scale = (F32(FP8_MAX[fmt]) / amax).astype(F32)
    scale_inv = (F32(1.0) / scale).astype(F32)
    return scale, scale_inv


# --------------------------------------------------------------------------- tensorwise / rowwise
def quantize_fp8_tensorwise(x: np.ndarray, fmt: str):
    """csrc/pytorch/quantization/quantization.cpp:44-90. Returns (q bytes, scale_inv 0-dim)."""
    x = np.asarray(x, dtype=F32)
    amax = _amax(x)
    scale, scale_inv = _scale_from_amax(amax, fmt, 1e-12)
    return _quant_clamp_encode(x, scale, fmt), np.asarray(scale_inv, dtype=F32).reshape(())


def quantize_fp8_rowwise(x: np.ndarray, fmt: str, axis: int):
    """quantization.cpp:110-208, quantization_rowwise.cu:59-137,188-237.
    Returns (q bytes same shape, scale_inv with `axis` reduced to 1)."""
    x = np.asarray(x, dtype=F32)
    axis = axis % x.ndim
    amax = _amax(x, axis=axis, keepdims=True)
    scale, scale_inv = _scale_from_amax(amax, fmt, 1e-12)
    return _quant_clamp_encode(x, scale, fmt), scale_inv


def dequantize_fp8(q: np.ndarray, scale_inv: np.ndarray, fmt: str) -> np.ndarray:
    """float(q) * scale_inv in fp32 (quantization.cpp:211-330)."""
    return (decode(q, fmt) * np.asarray(scale_inv, dtype=F32)).astype(F32)


# --------------------------------------------------------------------------- 128-blockwise
def quantize_fp8_blockwise(x: np.ndarray, fmt: str, axis: int, block: int = 128):
    """primus_turbo/triton/quantization/quant_blockwise.py:11-62.
    axis=1: scales [M, ceil(N/block)]; axis=0: scales [ceil(M/block), N]."""
    x = np.asarray(x, dtype=F32)
    M, N = x.shape
    if axis in (1, -1):
        nb = (N + block - 1) // block
        xp = np.zeros((M, nb * block), dtype=F32)
        xp[:, :N] = x
        blk = xp.reshape(M, nb, block)
        amax = _amax(blk, axis=2)
        scale, scale_inv = _scale_from_amax(amax, fmt, 1e-4)
        q = _quant_clamp_encode(blk, scale[:, :, None], fmt).reshape(M, nb * block)[:, :N]
        return np.ascontiguousarray(q), scale_inv
    mb = (M + block - 1) // block
    xp = np.zeros((mb * block, N), dtype=F32)
    xp[:M] = x
    blk = xp.reshape(mb, block, N)
    amax = _amax(blk, axis=1)
    scale, scale_inv = _scale_from_amax(amax, fmt, 1e-4)
    q = _quant_clamp_encode(blk, scale[:, None, :], fmt).reshape(mb * block, N)[:M]
    return np.ascontiguousarray(q), scale_inv


def quantize_fp8_blockwise_dual(x: np.ndarray, fmt: str, block: int = 128):
    """quant_blockwise.py:66-112: (q_row, s_row [M, N/b], q_col (not transposed), s_col [M/b, N])."""
    q_row, s_row = quantize_fp8_blockwise(x, fmt, 1, block)
    q_col, s_col = quantize_fp8_blockwise(x, fmt, 0, block)
    return q_row, s_row, q_col, s_col


def quantize_fp8_blockwise_weight(w: np.ndarray, fmt: str, block: int = 128):
    """One scale per block x block tile (quant_blockwise.py:119-156,
    quantization_blockwise.cu:248-334). w is [M,N] or [B,M,N]."""
    w = np.asarray(w, dtype=F32)
    squeeze = w.ndim == 2
    if squeeze:
        w = w[None]
    B, M, N = w.shape
    mb, nb = (M + block - 1) // block, (N + block - 1) // block
    wp = np.zeros((B, mb * block, nb * block), dtype=F32)
    wp[:, :M, :N] = w
    t = wp.reshape(B, mb, block, nb, block)
    amax = _amax(t, axis=(2, 4))
    scale, scale_inv = _scale_from_amax(amax, fmt, 1e-4)
    q = _quant_clamp_encode(t, scale[:, :, None, :, None], fmt).reshape(B, mb * block, nb * block)
    q = np.ascontiguousarray(q[:, :M, :N])
    if squeeze:
        return q[0], scale_inv[0]
    return q, scale_inv


def dequantize_fp8_blockwise(q, scale_inv, fmt: str, axis: int, block: int = 128):
    """quant_blockwise.py:163-234."""
    v = decode(q, fmt)
    M, N = v.shape
    if axis in (1, -1):
        s = np.repeat(scale_inv, block, axis=1)[:, :N]
    else:
        s = np.repeat(scale_inv, block, axis=0)[:M]
    return (v * s).astype(F32)


def dequantize_fp8_blockwise_weight(q, scale_inv, fmt: str, block: int = 128):
    v = decode(q, fmt)
    M, N = v.shape[-2:]
    s = np.repeat(np.repeat(scale_inv, block, axis=-2), block, axis=-1)[..., :M, :N]
    return (v * s).astype(F32)


def padded_group_offs(group_lens: np.ndarray, align: int = 128):
    """Per-group lengths rounded up to `align` and their exclusive prefix sums
    (quantization_blockwise.cu:18-36)."""
    lens = np.asarray(group_lens, dtype=np.int64)
    plens = (lens + align - 1) // align * align
    offs = np.zeros(len(lens) + 1, dtype=np.int64)
    offs[1:] = np.cumsum(plens)
    return plens, offs


def group_offs_from_lens(group_lens: np.ndarray) -> np.ndarray:
    """csrc/kernels/grouped_gemm/compute_group_offs.cu:15-32."""
    lens = np.asarray(group_lens, dtype=np.int64)
    offs = np.zeros(len(lens) + 1, dtype=np.int64)
    offs[1:] = np.cumsum(lens)
    return offs


def quantize_fp8_blockwise_segment_m(x: np.ndarray, fmt: str, group_lens: np.ndarray, block: int = 128):
    """Grouped row (1 x 128) + column (128 x 1 over each group's zero padded segment) quantization
    (quantization_blockwise.cu:60-215, quant_blockwise.py:238-327).

    Returns (q_row [M,N], q_col_padded [M + G*128, N], s_row [ceil(N/128), M] (transposed),
    s_col_padded [(M + G*128)/128, N], padded_lens [G], padded_offs [G+1]).  Rows of the padded
    buffers at or beyond padded_offs[G] are not written by the kernel; here they are zero.
    """
    x = np.asarray(x, dtype=F32)
    M, N = x.shape
    G = len(group_lens)
    offs = group_offs_from_lens(group_lens)
    plens, poffs = padded_group_offs(group_lens, block)
    m_alloc = M + G * block
    q_row, s_row = quantize_fp8_blockwise(x, fmt, 1, block)
    q_col = np.zeros((m_alloc, N), dtype=np.uint8)
    s_col = np.zeros((m_alloc // block, N), dtype=F32)
    for g in range(G):
        n = int(group_lens[g])
        if plens[g] == 0:
            continue
        seg = np.zeros((int(plens[g]), N), dtype=F32)
        seg[:n] = x[offs[g]:offs[g] + n]
        qs, ss = quantize_fp8_blockwise(seg, fmt, 0, block)
        q_col[poffs[g]:poffs[g + 1]] = qs
        s_col[poffs[g] // block:poffs[g + 1] // block] = ss
    return q_row, q_col, np.ascontiguousarray(s_row.T), s_col, plens, poffs


# --------------------------------------------------------------------------- MX (32-element, ue8m0)
def _rht16(v: np.ndarray) -> np.ndarray:
    """16-point Hadamard on the last axis (length multiple of 16), op order of
    quantization_mxfp4.cu:91-136: H4 inside each run of 4, then butterflies across the four
    runs (partner xor 1, then xor 2), then * 0.25."""
    shp = v.shape
    t = v.astype(F32).reshape(shp[:-1] + (shp[-1] // 16, 4, 4)).copy()
    v0, v1, v2, v3 = t[..., 0], t[..., 1], t[..., 2], t[..., 3]
    a0, a1, a2, a3 = v0 + v1, v0 - v1, v2 + v3, v2 - v3
    w = np.stack([a0 + a2, a1 + a3, a0 - a2, a1 - a3], axis=-1).astype(F32)  # [..., thread, i]
    for bit in (1, 2):
        idx = np.arange(4) ^ bit
        p = w[..., idx, :]
        neg = ((np.arange(4) & bit) != 0)[:, None]
        w = np.where(neg, p - w, p + w).astype(F32)
    w = (w * F32(0.25)).astype(F32)
    return w.reshape(shp)


def _mx_quant_rows(xr: np.ndarray, fmt: str, tile_amax, zero_scale_byte: int, use_rht: bool):
    """xr [R, C] float32 with C % 32 == 0: 32-element blocks along the last axis.
    tile_amax: optional [R, C/32] amax override (2D-block mode)."""
    R, C = xr.shape
    blk = xr.reshape(R, C // 32, 32).astype(F32)
    if use_rht:
        blk = _rht16(blk)
    amax = _amax(blk, axis=2) if tile_amax is None else tile_amax
    byte, scale = mx_scale_from_amax(amax, fmt)
    if zero_scale_byte != 0:
        byte = np.where(amax == 0, np.uint8(zero_scale_byte), byte)
        scale = np.where(amax == 0, F32(1.0), scale)
    s = scale[:, :, None]
    if fmt != E2M1:
        lim = (F32(FP8_MAX[fmt]) * s).astype(F32)
        blk = np.fmin(np.fmax(blk, -lim), lim)  # quantization_mxfp8.cu:131-136
    with np.errstate(divide="ignore", invalid="ignore"):
        v = (blk / s).astype(F32)
    v = np.where(s == 0, F32(0), v)  # scale byte 0: every |value| < 2^-126, convert gives 0
    codes = encode(v, fmt).reshape(R, C)
    return codes, byte


def _tile_amax_2d(xp: np.ndarray) -> np.ndarray:
    """amax over 32x32 tiles of a [R32, C32] padded array -> [R32/32, C32/32]."""
    R, C = xp.shape
    return _amax(xp.reshape(R // 32, 32, C // 32, 32), axis=(1, 3)).astype(F32)


def quantize_mx(x: np.ndarray, fmt: str, axis: int, use_2d_block: bool = False,
                use_rht: bool = False, zero_scale_byte: int = 0, align: int = 128):
    """MXFP8 (fmt e4m3/e5m2) or MXFP4 (fmt e2m1) quantization of a 2-D array.

    axis=1 (row-wise): data [M, N_pad] (fp4: packed [M, N_pad/2]), scale [M, N_pad/32].
    axis=0 (col-wise): data transposed [N, M_pad] (fp4: [N, M_pad/2]), scale [N, M_pad/32].
    Pads are ceil-to-128 and hold zeros (quantization.cpp:737-969, 511-734;
    quantization_mxfp8.cu:231-537; quantization_mxfp4.cu:292-629).
    """
    x = np.asarray(x, dtype=F32)
    M, N = x.shape
    assert N % 32 == 0, "N must be divisible by 32"
    M_pad, N_pad = _ceil_to(M, align), _ceil_to(N, align)
    xp = np.zeros((M_pad, N_pad), dtype=F32)
    xp[:M, :N] = x
    tile = _tile_amax_2d(xp) if use_2d_block else None
    if axis in (1, -1):
        ta = np.repeat(tile, 32, axis=0)[:M] if use_2d_block else None
        codes, byte = _mx_quant_rows(xp[:M], fmt, ta, zero_scale_byte, use_rht)
    else:
        xt = np.ascontiguousarray(xp[:, :N].T)
        ta = np.repeat(tile.T, 32, axis=0)[:N] if use_2d_block else None
        codes, byte = _mx_quant_rows(xt, fmt, ta, zero_scale_byte, use_rht)
    if fmt == E2M1:
        codes = pack_e2m1(codes)
    return codes, byte


def quantize_mx_dual(x, fmt, row_2d=False, col_2d=False, row_rht=False, col_rht=False):
    q_r, s_r = quantize_mx(x, fmt, 1, row_2d, row_rht)
    q_c, s_c = quantize_mx(x, fmt, 0, col_2d, col_rht)
    return q_r, s_r, q_c, s_c


def quantize_mx_batched(x, fmt, axis, use_2d_block=False, use_rht=False):
    """3-D input [G, M, N]; axis 2 = row-wise, axis 1 = col-wise (quantization.cpp:884-900)."""
    outs = [quantize_mx(x[g], fmt, 1 if axis in (2, -1) else 0, use_2d_block, use_rht) for g in range(x.shape[0])]
    return np.stack([o[0] for o in outs]), np.stack([o[1] for o in outs])


def dequantize_mx(q: np.ndarray, scale: np.ndarray, fmt: str) -> np.ndarray:
    """decode(q) * 2^(byte-127) (dequantization_mxfp8.cu, dequantization_mxfp4.cu:26-27,111)."""
    codes = unpack_e2m1(q) if fmt == E2M1 else q
    v = decode(codes, fmt)
    s = np.repeat(e8m0_decode(scale), 32, axis=-1)
    return (v * s).astype(F32)


def quantize_mx_grouped(x: np.ndarray, fmt: str, group_lens, axis: int, use_2d_block=False,
                        use_rht=False, row_align: int = 32, col_align: int = 128):
    """Grouped MX quantization of x [total_M, N] (quantization_mxfp8.cu:979-1709,
    quantization_mxfp4.cu:1327-2045).  Zero-amax blocks get scale byte 127.

    axis=1: FP8 -> each group's rows padded to `row_align` (pad rows are NOT written by the
    kernel; zero here), data [sum(pad_r), N_pad], scale [sum(pad_r), N_pad/32].
            FP4 -> tight (row i = input row i): pass row_align=1.
    axis=0: each group's segment zero-padded to `col_align` rows and transposed:
            data [N, sum(pad_c)], scale [N, sum(pad_c)/32].
    Returns (data, scale, padded_lens, padded_offs).
    """
    x = np.asarray(x, dtype=F32)
    M, N = x.shape
    offs = group_offs_from_lens(group_lens)
    G = len(group_lens)
    N_pad = _ceil_to(N, 128)
    if axis in (1, -1):
        plens, poffs = padded_group_offs(group_lens, row_align)
        tot = int(poffs[-1])
        data = np.zeros((tot, N_pad if fmt != E2M1 else N_pad // 2), dtype=np.uint8)
        scale = np.full((tot, N_pad // 32), 127, dtype=np.uint8)
        for g in range(G):
            n = int(group_lens[g])
            if n == 0:
                continue
            seg = x[offs[g]:offs[g] + n]
            q, s = _grouped_seg(seg, fmt, 1, use_2d_block, use_rht)
            data[poffs[g]:poffs[g] + n] = q
            scale[poffs[g]:poffs[g] + n] = s
        return data, scale, plens, poffs
    plens, poffs = padded_group_offs(group_lens, col_align)
    tot = int(poffs[-1])
    data = np.zeros((N, tot if fmt != E2M1 else tot // 2), dtype=np.uint8)
    scale = np.full((N, tot // 32), 127, dtype=np.uint8)
    for g in range(G):
        n = int(group_lens[g])
        if plens[g] == 0:
            continue
        seg = np.zeros((int(plens[g]), N), dtype=F32)
        seg[:n] = x[offs[g]:offs[g] + n]
        q, s = _grouped_seg(seg, fmt, 0, use_2d_block, use_rht)
        c0, c1 = int(poffs[g]), int(poffs[g + 1])
        if fmt == E2M1:
            data[:, c0 // 2:c1 // 2] = q[:, :(c1 - c0) // 2]
        else:
            data[:, c0:c1] = q[:, :c1 - c0]
        scale[:, c0 // 32:c1 // 32] = s[:, :(c1 - c0) // 32]
    return data, scale, plens, poffs


def _grouped_seg(seg, fmt, axis, use_2d_block, use_rht):
    return quantize_mx(seg, fmt, axis, use_2d_block, use_rht, zero_scale_byte=127)
