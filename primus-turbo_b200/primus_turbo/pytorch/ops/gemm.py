"""gemm: BF16 / FP16 GEMM with autograd, on the tcgen05 kernels of the FP8 path run with 16-bit operands.

Operator surface and data flow follow primus_turbo/pytorch/ops/gemm.py of the reference (GemmFunction, gemm).
"""
from typing import Optional, Union

import torch

from ..kernels.gemm.gemm_impl import gemm_accum_impl, gemm_impl
from .utils import _get_dummy_wgrad, _setup_fused_grad_accum

__all__ = ["gemm"]


class GemmFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, a, b, trans_a, trans_b, out_dtype, fuse_bgrad_accum_pattern=None):
        assert a.dim() == 2 and b.dim() == 2, "Only 2D GEMM is supported"
        fuse, main_grad = _setup_fused_grad_accum(b, fuse_bgrad_accum_pattern)
        out = gemm_impl(a, trans_a, b, trans_b, out_dtype, False)
        ctx.save_for_backward(a, b)
        ctx.trans_a, ctx.trans_b, ctx.fuse, ctx.main_grad = trans_a, trans_b, fuse, main_grad
        return out

    @staticmethod
    def backward(ctx, grad_out):
        a, b = ctx.saved_tensors
        grad_out = grad_out.contiguous()
        if grad_out.dtype != a.dtype:
            grad_out = grad_out.to(a.dtype)
        grad_a = gemm_impl(grad_out, False, b, not ctx.trans_b, a.dtype, ctx.trans_a)      # grad_out . b^T
        if ctx.fuse:
            gemm_accum_impl(a, not ctx.trans_a, grad_out, False, b.dtype, ctx.trans_b, out=ctx.main_grad)
            grad_b = _get_dummy_wgrad(b.shape, b.dtype, device=b.device)
        else:
            grad_b = gemm_impl(a, not ctx.trans_a, grad_out, False, b.dtype, ctx.trans_b)  # a^T . grad_out
        return grad_a, grad_b, None, None, None, None


def gemm(a: torch.Tensor, b: torch.Tensor, trans_a: bool = False, trans_b: bool = False, out_dtype: Optional[torch.dtype] = None,
         fuse_bgrad_accum_pattern: Union[None, str] = None) -> torch.Tensor:
    """out = op(a) . op(b) for 2-D bf16 / fp16 tensors; fp32 accumulate."""
    if out_dtype is None:
        out_dtype = torch.result_type(a, b)
    return GemmFunction.apply(a, b, trans_a, trans_b, out_dtype, fuse_bgrad_accum_pattern)
