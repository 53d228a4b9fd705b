"""BF16 / FP16 grouped GEMMs over the C ABI.

Call shapes follow primus_turbo::grouped_gemm_impl, grouped_gemm_variable_k_impl and grouped_gemm_variable_k_accum_impl
of the reference (primus_turbo/pytorch/kernels/grouped_gemm/grouped_gemm_impl.py).  Group lengths stay on the device.
"""
from typing import Optional

import torch

from .. import _native as nv
from ..quantization.quantization_impl import compute_padded_group_offs, grouped_transpose_pad, transpose_batched


def grouped_gemm_impl(a: torch.Tensor, b: torch.Tensor, group_lens: torch.Tensor, group_offs: torch.Tensor, trans_a: bool = False,
                      trans_b: bool = False, num_cu: Optional[int] = None, default_backend: int = 0, maybe_pre_sync: bool = False,
                      schedule: str = "static") -> torch.Tensor:
    """out[rows of group g] = a[rows of group g] . op(b[g]); a [sum(lens), K], b [G, N, K] (trans_b) or [G, K, N]."""
    nv.require_cuda(a, b, group_lens, group_offs)
    assert not trans_a, "grouped GEMM takes a row-major activation (trans_a=False)"
    assert a.dim() == 2 and b.dim() == 3
    assert a.dtype == b.dtype and a.dtype in (torch.bfloat16, torch.float16), "a and b must both be bf16 or fp16"
    assert schedule == "static", "only the static persistent schedule is provided"
    a = a.contiguous()
    b_km = b.contiguous() if trans_b else transpose_batched(b)   # [G, N, K]
    G, N, K = b_km.shape
    rows = a.shape[0]
    assert a.shape[1] == K and K % 8 == 0, "the contraction length must match and be a multiple of 8"
    offs = group_offs.to(torch.int64).contiguous()
    out = torch.empty((rows, N), dtype=a.dtype, device=a.device)
    st = nv.status_word(a.device)
    with nv.on_device(a.device):
        nv.check(nv.lib().pt_zero_rows_from(nv.ptr(out), rows, N * out.element_size(), nv.ptr(offs[G:]), nv.stream(a.device)),
                 "zero_rows_from")
        nv.check(nv.lib().pt_grouped_gemm(nv.ptr(a), nv.ptr(b_km), nv.src_code(a.dtype), nv.ptr(out), nv.src_code(out.dtype), rows, N, K,
                                           nv.ptr(offs), G, 0.0, int(num_cu) if num_cu else 0, nv.ptr(st), nv.stream(a.device)),
                 "grouped_gemm")
    nv.poll_status(out.device)
    return out


def _variable_k(a, b, group_lens, group_offs, trans_a, trans_b, trans_c, num_cu, out=None):
    nv.require_cuda(a, b, group_lens, group_offs)
    assert trans_a and not trans_b, "variable-K takes token-major operands (trans_a=True, trans_b=False)"
    assert a.dim() == 2 and b.dim() == 2 and a.shape[0] == b.shape[0]
    assert a.dtype == b.dtype and a.dtype in (torch.bfloat16, torch.float16)
    G = group_lens.numel()
    _, poffs = compute_padded_group_offs(group_lens, 128)
    a_t = grouped_transpose_pad(a, group_offs, poffs)   # [Ka, T]: each group's tokens in a zero-filled 128-aligned segment
    b_t = grouped_transpose_pad(b, group_offs, poffs)   # [Nb, T]
    lhs, rhs = (b_t, a_t) if trans_c else (a_t, b_t)
    R, T = lhs.shape
    Nn = rhs.shape[0]
    beta = 0.0 if out is None else 1.0
    if out is None:
        out = torch.empty((G, R, Nn), dtype=a.dtype, device=a.device)
    else:
        assert out.is_contiguous() and tuple(out.shape) == (G, R, Nn)
    st = nv.status_word(a.device)
    with nv.on_device(a.device):
        nv.check(nv.lib().pt_grouped_gemm_variable_k(nv.ptr(lhs), nv.ptr(rhs), nv.src_code(lhs.dtype), nv.ptr(out),
                                                      nv.src_code(out.dtype), R, Nn, T, nv.ptr(poffs), G, beta,
                                                      int(num_cu) if num_cu else 0, nv.ptr(st), nv.stream(a.device)),
                 "grouped_gemm_variable_k")
    nv.poll_status(out.device)
    return out


def grouped_gemm_variable_k_impl(a, b, group_lens, group_offs, trans_a: bool = True, trans_b: bool = False, trans_c: bool = False,
                                 num_cu: Optional[int] = None, default_backend: int = 0, schedule: str = "static"):
    """Per group g: C[g] = a[rows of g]^T . b[rows of g] -> [G, Ka, Nb] ([G, Nb, Ka] when trans_c)."""
    return _variable_k(a, b, group_lens, group_offs, trans_a, trans_b, trans_c, num_cu)


def grouped_gemm_variable_k_accum_impl(a, b, group_lens, group_offs, trans_a: bool = True, trans_b: bool = False,
                                       trans_c: bool = False, num_cu: Optional[int] = None, default_backend: int = 0,
                                       out: Optional[torch.Tensor] = None, schedule: str = "static"):
    """out[g] += ... in place."""
    assert out is not None
    return _variable_k(a, b, group_lens, group_offs, trans_a, trans_b, trans_c, num_cu, out=out)
