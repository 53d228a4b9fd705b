"""CPU restatement (numpy, integer index arithmetic) of the reference's pre-shuffled MX layouts.  TEST INFRASTRUCTURE ONLY:
the product never imports this module.

Follows csrc/include/primus_turbo/device/shuffle.cuh:39-48 (`compute_shuffle_scale_index`) and :61-80
(`compute_shuffled_index`), with the padding of csrc/pytorch/shuffle/shuffle.cpp:33-45 (scale rows to a multiple of 256,
scale columns to a multiple of 8, padding bytes 0) and the divisibility rules of :62-66 (rows % 16, row bytes % 32).
Pinned by hand-computed positions in tests/test_oracle_codecs.py (the reference's own test only compares its two code
paths with each other: tests/pytorch/ops/test_quantization.py:500-560).
"""
import numpy as np


def shuffle_scale(scale: np.ndarray) -> np.ndarray:
    """scale uint8 [M, N] -> uint8 [ceil(M, 256), ceil(N, 8)]."""
    M, N = scale.shape
    m_pad, n_pad = -(-M // 256) * 256, -(-N // 8) * 8
    out = np.zeros(m_pad * n_pad, dtype=np.uint8)
    row, col = np.meshgrid(np.arange(M), np.arange(N), indexing="ij")
    i0, i1, i2 = row >> 5, (row >> 4) & 1, row & 15
    i3, i4, i5 = col >> 3, (col >> 2) & 1, col & 3
    idx = (i0 * (n_pad >> 3) << 8) + (i3 << 8) + (i5 << 6) + (i2 << 2) + (i4 << 1) + i1
    out[idx.ravel()] = scale.ravel()
    return out.reshape(m_pad, n_pad)


def shuffle_codes(codes: np.ndarray) -> np.ndarray:
    """codes uint8 [M, row_bytes] (packed e2m1 pairs or fp8 bytes), M % 16 == 0, row_bytes % 32 == 0 -> same shape."""
    M, K = codes.shape
    assert M % 16 == 0 and K % 32 == 0
    row, col = np.meshgrid(np.arange(M), np.arange(K), indexing="ij")
    cib = col & 31
    idx = (row >> 4) * (K << 4) + (col >> 5) * 512 + (cib >> 4) * 256 + (row & 15) * 16 + (cib & 15)
    out = np.empty(M * K, dtype=np.uint8)
    out[idx.ravel()] = codes.ravel()
    return out.reshape(M, K)
