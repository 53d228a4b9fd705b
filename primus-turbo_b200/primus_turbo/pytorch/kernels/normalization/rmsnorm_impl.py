"""RMSNorm forward / backward (plain and fused-residual) over the C ABI.  Mirrors
primus_turbo/pytorch/kernels/normalization/rmsnorm_impl.py of the reference, without its launch-tuning return values."""
from typing import Optional, Tuple

import torch

from .. import _native as nv


def _fwd(x2, residual2, gamma, eps, zero_centered, want_y=True):
    rows, H = x2.shape
    y = torch.empty_like(x2) if want_y else None
    xpr = torch.empty_like(x2) if residual2 is not None else None
    rstd = torch.empty((rows,), dtype=torch.float32, device=x2.device)
    with nv.on_device(x2.device):
        nv.check(nv.lib().pt_rmsnorm_fwd(nv.ptr(x2), nv.ptr(residual2), nv.ptr(gamma), nv.src_code(x2.dtype), float(eps), int(bool(zero_centered)),
                                         rows, H, nv.ptr(y), nv.ptr(xpr), nv.ptr(rstd), nv.stream(x2.device)), "rmsnorm_fwd")
    return y, xpr, rstd


def rmsnorm_fwd_impl(x: torch.Tensor, gamma: torch.Tensor, eps: float, zero_centered: bool = False):
    """-> (y [rows, H], x as [rows, H], rstd fp32 [rows])."""
    nv.require_cuda(x, gamma)
    assert gamma.dtype == x.dtype, "rmsnorm: gamma must have the dtype of x"
    x2 = x.reshape(-1, x.shape[-1]).contiguous()
    y, _, rstd = _fwd(x2, None, gamma.contiguous(), eps, zero_centered)
    return y, x2, rstd


def rmsnorm_fwd_residual_impl(x: torch.Tensor, residual: torch.Tensor, gamma: torch.Tensor, eps: float):
    """-> (y, x + residual rounded to the dtype, rstd)."""
    nv.require_cuda(x, residual, gamma)
    assert gamma.dtype == x.dtype == residual.dtype
    x2 = x.reshape(-1, x.shape[-1]).contiguous()
    r2 = residual.reshape(-1, x.shape[-1]).contiguous()
    return _fwd(x2, r2, gamma.contiguous(), eps, False)


def rmsnorm_stats_impl(x: torch.Tensor, eps: float) -> torch.Tensor:
    """rstd alone (fp32 [rows]): the row statistic a fused normalise-and-quantize kernel consumes."""
    nv.require_cuda(x)
    x2 = x.reshape(-1, x.shape[-1]).contiguous()
    return _fwd(x2, None, None, eps, False, want_y=False)[2]


def _bwd(dy, dxpr, x2, gamma, rstd, zero_centered) -> Tuple[torch.Tensor, torch.Tensor]:
    rows, H = x2.shape
    dy2 = dy.reshape(rows, H).contiguous()
    dxpr2 = None if dxpr is None else dxpr.reshape(rows, H).contiguous()
    dx = torch.empty_like(x2)
    dgamma = torch.empty_like(gamma)
    lib = nv.lib()
    parts = lib.pt_rmsnorm_bwd_parts(rows)
    partial = torch.empty((parts, H), dtype=torch.float32, device=x2.device)
    with nv.on_device(x2.device):
        nv.check(lib.pt_rmsnorm_bwd(nv.ptr(dy2), nv.ptr(dxpr2), nv.ptr(x2), nv.ptr(gamma), nv.ptr(rstd), nv.src_code(x2.dtype),
                                    int(bool(zero_centered)), rows, H, nv.ptr(dx), nv.ptr(dgamma), nv.ptr(partial), parts,
                                    nv.stream(x2.device)), "rmsnorm_bwd")
    return dx, dgamma


def rmsnorm_bwd_impl(grad_out, x2, gamma, rstd, zero_centered: bool = False):
    return _bwd(grad_out, None, x2, gamma.contiguous(), rstd, zero_centered)


def rmsnorm_bwd_residual_impl(grad_y, grad_xpr: Optional[torch.Tensor], x_plus_r, gamma, rstd):
    return _bwd(grad_y, grad_xpr, x_plus_r, gamma.contiguous(), rstd, False)
