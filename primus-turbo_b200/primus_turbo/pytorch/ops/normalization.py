"""rmsnorm / rmsnorm_residual with autograd; interface of primus_turbo/pytorch/ops/normalization.py of the reference."""
from typing import Tuple

import torch

from ..kernels.normalization.rmsnorm_impl import (
    rmsnorm_bwd_impl,
    rmsnorm_bwd_residual_impl,
    rmsnorm_fwd_impl,
    rmsnorm_fwd_residual_impl,
)

__all__ = ["rmsnorm", "rmsnorm_residual"]


class _RMSNormFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, gamma, eps=1e-6, zero_centered=False):
        assert x.is_cuda and gamma.is_cuda, "rmsnorm: x and gamma must be CUDA tensors"
        H = gamma.shape[0]
        assert x.shape[-1] == H, f"rmsnorm: last dim of x ({x.shape[-1]}) must equal gamma.shape[0] ({H})"
        y, x2, rstd = rmsnorm_fwd_impl(x, gamma, eps, zero_centered)
        ctx.save_for_backward(x2, gamma, rstd)
        ctx.zero_centered, ctx.orig_shape = zero_centered, x.shape
        return y.reshape(x.shape)

    @staticmethod
    def backward(ctx, grad_out):
        x2, gamma, rstd = ctx.saved_tensors
        dx, dg = rmsnorm_bwd_impl(grad_out, x2, gamma, rstd, ctx.zero_centered)
        return dx.reshape(ctx.orig_shape), dg, None, None


class _RMSNormResidualFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, residual, gamma, eps=1e-6):
        assert x.is_cuda and residual.is_cuda and gamma.is_cuda, "rmsnorm_residual: x, residual and gamma must be CUDA tensors"
        assert x.shape == residual.shape, f"rmsnorm_residual: shape mismatch {tuple(x.shape)} vs {tuple(residual.shape)}"
        assert x.shape[-1] == gamma.shape[0]
        y, x_plus_r, rstd = rmsnorm_fwd_residual_impl(x, residual, gamma, eps)
        ctx.save_for_backward(x_plus_r, gamma, rstd)
        ctx.orig_shape = x.shape
        return y.reshape(x.shape), x_plus_r.reshape(x.shape)

    @staticmethod
    def backward(ctx, grad_y, grad_xpr):
        x_plus_r, gamma, rstd = ctx.saved_tensors
        dx, dg = rmsnorm_bwd_residual_impl(grad_y, grad_xpr, x_plus_r, gamma, rstd)
        dx = dx.reshape(ctx.orig_shape)
        return dx, dx, dg, None   # the add sends the same gradient to x and to the residual


def rmsnorm(x: torch.Tensor, gamma: torch.Tensor, eps: float = 1e-6, zero_centered: bool = False) -> torch.Tensor:
    """y = x * rsqrt(mean(x^2, -1) + eps) * (gamma, or 1 + gamma when zero_centered); statistics in fp32."""
    return _RMSNormFunction.apply(x, gamma, eps, zero_centered)


def rmsnorm_residual(x: torch.Tensor, residual: torch.Tensor, gamma: torch.Tensor, eps: float = 1e-6) -> Tuple[torch.Tensor, torch.Tensor]:
    """(rmsnorm(x + residual), x + residual) in one pass over the row."""
    return _RMSNormResidualFunction.apply(x, residual, gamma, eps)
