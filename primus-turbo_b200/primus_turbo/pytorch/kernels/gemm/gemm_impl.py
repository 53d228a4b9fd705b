"""BF16 / FP16 dense GEMM over the C ABI.

Same call shape as primus_turbo::gemm_impl / gemm_accum_impl of the reference
(primus_turbo/pytorch/kernels/gemm/gemm_impl.py).  The CUDA kernel is the FP8 one run with kind::f16 instructions:
C = A . B^T with both operands K-major; the other (trans_a, trans_b, trans_c) combinations swap the operands
(trans_c) or transpose the 16-bit elements first.
"""
import torch

from .. import _native as nv
from ..quantization.quantization_impl import transpose_2d


def _k_major16(x, trans):
    """x as [rows, K] with K a multiple of 8 (a 16-byte row pitch): x itself, its transpose, zero padded if ragged."""
    x = x.contiguous()
    y = transpose_2d(x) if trans else x
    K = y.shape[1]
    if K % 8 == 0:
        return y
    z = torch.zeros((y.shape[0], (K + 7) // 8 * 8), dtype=y.dtype, device=y.device)
    z[:, :K] = y
    return z


def _launch(a_km, b_km, out, beta):
    M, K = a_km.shape
    N = b_km.shape[0]
    assert b_km.shape[1] == K, f"contraction mismatch: {tuple(a_km.shape)} vs {tuple(b_km.shape)}"
    st = nv.status_word(out.device)
    with nv.on_device(out.device):
        nv.check(nv.lib().pt_gemm(nv.ptr(a_km), nv.ptr(b_km), nv.src_code(a_km.dtype), nv.ptr(out), nv.src_code(out.dtype), M, N, K,
                                   float(beta), nv.ptr(st), nv.stream(out.device)), "gemm")
    nv.poll_status(out.device)
    return out


def _gemm(a, trans_a, b, trans_b, out_dtype, trans_c, out=None):
    nv.require_cuda(a, b)
    assert a.dim() == 2 and b.dim() == 2, "Only 2D tensors are supported"
    assert a.dtype == b.dtype and a.dtype in (torch.bfloat16, torch.float16), "a and b must both be bf16 or fp16"
    a_km = _k_major16(a, trans_a)        # [M, K]
    b_km = _k_major16(b, not trans_b)    # [N, K]
    M, N = a_km.shape[0], b_km.shape[0]
    beta = 0.0 if out is None else 1.0
    if out is None:
        out = torch.empty((N, M) if trans_c else (M, N), dtype=out_dtype, device=a.device)
    else:
        assert out.is_contiguous() and tuple(out.shape) == ((N, M) if trans_c else (M, N))
    return _launch(b_km, a_km, out, beta) if trans_c else _launch(a_km, b_km, out, beta)


def gemm_impl(a: torch.Tensor, trans_a: bool, b: torch.Tensor, trans_b: bool, out_dtype: torch.dtype, trans_c: bool,
              default_backend: int = 0) -> torch.Tensor:
    """op(a) . op(b) (transposed when trans_c), fp32 accumulate, output in out_dtype."""
    return _gemm(a, trans_a, b, trans_b, out_dtype, trans_c)


def gemm_accum_impl(a: torch.Tensor, trans_a: bool, b: torch.Tensor, trans_b: bool, out_dtype: torch.dtype, trans_c: bool,
                    out: torch.Tensor, default_backend: int = 0) -> torch.Tensor:
    """out += op(a) . op(b) in place (the fused main_grad accumulation of the wgrad)."""
    return _gemm(a, trans_a, b, trans_b, out.dtype, trans_c, out=out)
