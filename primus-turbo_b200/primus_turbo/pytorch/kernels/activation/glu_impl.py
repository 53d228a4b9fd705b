"""Gated activations with routing probabilities over the C ABI.  Function names and argument order follow
primus_turbo/pytorch/kernels/activation/{swiglu,geglu}_impl.py of the reference."""
from typing import Optional, Tuple

import torch

from .. import _native as nv

ACT_CODES = {"silu": 0, "gelu": 1}


def glu_fwd_with_probs(x: torch.Tensor, probs: torch.Tensor, row_mask: Optional[torch.Tensor], act: str) -> torch.Tensor:
    """x [tokens, 2H], probs fp32 [tokens] -> [tokens, H] = act(x[:, :H]) * x[:, H:] * probs."""
    nv.require_cuda(x, probs, row_mask)
    tokens, h2 = x.shape
    assert h2 % 2 == 0
    x, probs = x.contiguous(), probs.contiguous().view(-1)
    out = torch.empty((tokens, h2 // 2), dtype=x.dtype, device=x.device)
    with nv.on_device(x.device):
        nv.check(nv.lib().pt_glu_fwd(nv.ptr(x), nv.src_code(x.dtype), nv.ptr(probs), nv.ptr(row_mask), tokens, h2 // 2, ACT_CODES[act],
                                     nv.ptr(out), nv.stream(x.device)), "glu_fwd")
    return out


def glu_bwd_with_probs(grad_out: torch.Tensor, x: torch.Tensor, probs: torch.Tensor, row_mask: Optional[torch.Tensor],
                       act: str) -> Tuple[torch.Tensor, torch.Tensor]:
    """(grad_x [tokens, 2H], grad_probs fp32 [tokens])."""
    nv.require_cuda(grad_out, x, probs, row_mask)
    tokens, h = grad_out.shape
    grad_out, x, probs = grad_out.contiguous(), x.contiguous(), probs.contiguous().view(-1)
    assert tuple(x.shape) == (tokens, 2 * h) and grad_out.dtype == x.dtype
    grad_x = torch.empty_like(x)
    grad_probs = torch.empty((tokens,), dtype=torch.float32, device=x.device)
    with nv.on_device(x.device):
        nv.check(nv.lib().pt_glu_bwd(nv.ptr(grad_out), nv.ptr(x), nv.src_code(x.dtype), nv.ptr(probs), nv.ptr(row_mask), tokens, h,
                                     ACT_CODES[act], nv.ptr(grad_x), nv.ptr(grad_probs), nv.stream(x.device)), "glu_bwd")
    return grad_x, grad_probs


def swiglu_fwd_with_probs(x, probs, row_mask=None):
    return glu_fwd_with_probs(x, probs, row_mask, "silu")


def swiglu_bwd_with_probs(grad_out, x, probs, row_mask=None):
    return glu_bwd_with_probs(grad_out, x, probs, row_mask, "silu")


def geglu_fwd_with_probs(x, probs, row_mask=None):
    return glu_fwd_with_probs(x, probs, row_mask, "gelu")


def geglu_bwd_with_probs(grad_out, x, probs, row_mask=None):
    return glu_bwd_with_probs(grad_out, x, probs, row_mask, "gelu")
