"""grouped_gemm: BF16 / FP16 MoE grouped GEMM with autograd.

Operator surface and data flow follow primus_turbo/pytorch/ops/grouped_gemm.py of the reference (GroupedGemmFunc,
grouped_gemm).  Group lengths are never read on the host.
"""
from typing import Optional, Union

import torch

from ..kernels.grouped_gemm.grouped_gemm_impl import (grouped_gemm_impl, grouped_gemm_variable_k_accum_impl,
                                                      grouped_gemm_variable_k_impl)
from ..kernels.grouped_gemm.grouped_gemm_utils import group_offs_from_lens
from .utils import _get_dummy_wgrad, _setup_fused_grad_accum

__all__ = ["grouped_gemm"]


class GroupedGemmFunc(torch.autograd.Function):
    @staticmethod
    def forward(ctx, a, b, group_lens, group_offs, trans_b, num_cu, schedule="static", fuse_bgrad_accum_pattern=None):
        fuse, main_grad = _setup_fused_grad_accum(b, fuse_bgrad_accum_pattern)
        out = grouped_gemm_impl(a, b, group_lens, group_offs, trans_a=False, trans_b=trans_b, num_cu=num_cu, schedule=schedule)
        ctx.save_for_backward(a, b, group_lens, group_offs)
        ctx.trans_b, ctx.num_cu, ctx.schedule, ctx.fuse, ctx.main_grad = trans_b, num_cu, schedule, fuse, main_grad
        return out

    @staticmethod
    def backward(ctx, grad_out):
        a, b, group_lens, group_offs = ctx.saved_tensors
        grad_out = grad_out.contiguous()
        grad_a = grouped_gemm_impl(grad_out, b, group_lens, group_offs, trans_a=False, trans_b=not ctx.trans_b, num_cu=ctx.num_cu,
                                   schedule=ctx.schedule)
        # grad_b[g] = a[g]^T . grad_out[g] -> [G, K, N]; transposed ([G, N, K]) when b is stored that way
        if ctx.fuse:
            grouped_gemm_variable_k_accum_impl(a, grad_out, group_lens, group_offs, trans_a=True, trans_b=False, trans_c=ctx.trans_b,
                                               num_cu=ctx.num_cu, out=ctx.main_grad, schedule=ctx.schedule)
            grad_b = _get_dummy_wgrad(b.shape, b.dtype, device=b.device)
        else:
            grad_b = grouped_gemm_variable_k_impl(a, grad_out, group_lens, group_offs, trans_a=True, trans_b=False,
                                                  trans_c=ctx.trans_b, num_cu=ctx.num_cu, schedule=ctx.schedule)
        return grad_a, grad_b, None, None, None, None, None, None


def grouped_gemm(a: torch.Tensor, b: torch.Tensor, group_lens: torch.Tensor, group_offs: Optional[torch.Tensor] = None,
                 trans_b: bool = False, num_cu: Optional[int] = None, schedule: str = "static",
                 fuse_bgrad_accum_pattern: Union[None, str] = None) -> torch.Tensor:
    """out[rows of group g] = a[rows of group g] . op(b[g]); a [sum(group_lens), K], b [G, K, N] or [G, N, K] (trans_b);
    group_lens int64 [G] on the device.  Only the static schedule exists here; num_cu caps the persistent CTAs."""
    if schedule != "static":
        raise ValueError("only schedule='static' is provided (the work-stealing variants are AMD XCD-specific)")
    if group_offs is None:
        group_offs = group_offs_from_lens(group_lens)
    return GroupedGemmFunc.apply(a, b, group_lens, group_offs, trans_b, num_cu, schedule, fuse_bgrad_accum_pattern)
