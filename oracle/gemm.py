"""fp32 reference GEMMs the CUDA GEMMs are checked against (test infrastructure).

GEMM parity is a tolerance, not bit-exactness: relative Frobenius error against
C_ref = dequant(qA) . dequant(qB)^T accumulated in fp32
(tests/pytorch/ref/gemm_ref.py:13-24, tests/pytorch/ref/quantization_ref.py:59-68).
"""
from __future__ import annotations

import numpy as np

F32 = np.float32


def gemm_nt(a: np.ndarray, b: np.ndarray) -> np.ndarray:
    """C[M,N] = A[M,K] . B[N,K]^T in fp32."""
    return np.matmul(np.asarray(a, dtype=F32), np.asarray(b, dtype=F32).T).astype(F32)


def gemm_blockwise_nt(qa_f32, sa, qb_f32, sb, block: int = 128) -> np.ndarray:
    """Blockwise accumulate exactly as the reference kernel orders it: per 128-K block
    acc += dot_kblock * (sa[m,kb] * sb[n/128,kb])
    (primus_turbo/triton/gemm/gemm_fp8_kernel.py:974-983).
    qa_f32 [M,K], sa [M,K/128], qb_f32 [N,K], sb [N/128,K/128]."""
    M, K = qa_f32.shape
    N = qb_f32.shape[0]
    acc = np.zeros((M, N), dtype=F32)
    sbn = np.repeat(sb, block, axis=0)[:N]
    for kb in range((K + block - 1) // block):
        k0, k1 = kb * block, min(K, (kb + 1) * block)
        part = np.matmul(qa_f32[:, k0:k1].astype(F32), qb_f32[:, k0:k1].astype(F32).T)
        acc += part * (sa[:, kb][:, None] * sbn[:, kb][None, :]).astype(F32)
    return acc


def grouped_gemm_nt(a: np.ndarray, b: np.ndarray, group_lens) -> np.ndarray:
    """C[offs[g]:offs[g+1]] = A[offs[g]:offs[g+1]] . B[g]^T   (gemm_ref.py:13-24). b is [G,N,K]."""
    outs, start = [], 0
    for g, n in enumerate(np.asarray(group_lens, dtype=np.int64)):
        outs.append(gemm_nt(a[start:start + n], b[g]))
        start += int(n)
    return np.concatenate(outs, axis=0) if outs else np.zeros((0, b.shape[1]), dtype=F32)


def grouped_gemm_variable_k(lhs: np.ndarray, rhs: np.ndarray, group_lens) -> np.ndarray:
    """C[g] = LHS[seg g]^T . RHS[seg g] -> [G, lhs_cols, rhs_cols]   (gemm_ref.py:27-41)."""
    G = len(group_lens)
    out = np.zeros((G, lhs.shape[1], rhs.shape[1]), dtype=F32)
    start = 0
    for g, n in enumerate(np.asarray(group_lens, dtype=np.int64)):
        n = int(n)
        if n:
            out[g] = np.matmul(lhs[start:start + n].T.astype(F32), rhs[start:start + n].astype(F32))
        start += n
    return out


def rel_frobenius(c: np.ndarray, c_ref: np.ndarray) -> float:
    c = np.asarray(c, dtype=np.float64)
    c_ref = np.asarray(c_ref, dtype=np.float64)
    d = np.linalg.norm(c_ref)
    return float(np.linalg.norm(c - c_ref) / d) if d > 0 else float(np.linalg.norm(c))


def snr_db(c: np.ndarray, c_ref: np.ndarray) -> float:
    """Signal-to-noise ratio used by the reference tests (tests/pytorch/test_utils.py)."""
    c = np.asarray(c, dtype=np.float64)
    c_ref = np.asarray(c_ref, dtype=np.float64)
    noise = np.sum((c - c_ref) ** 2)
    sig = np.sum(c_ref ** 2)
    return float(10 * np.log10(sig / max(noise, 1e-300)))
