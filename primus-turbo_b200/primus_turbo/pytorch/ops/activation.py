"""swiglu_with_probs / geglu_with_probs: gated activations scaled by the routing probability of each token, with autograd.
Same interface and checks as primus_turbo/pytorch/ops/activation.py:23-80 of the reference."""
from typing import Union

import torch

from ..kernels.activation.glu_impl import glu_bwd_with_probs, glu_fwd_with_probs

__all__ = ["swiglu_with_probs", "geglu_with_probs"]

SUPPORTED_ACT_TYPES = ["silu", "gelu"]


class GLUWithProbs(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, probs, row_mask, act_type):
        x_shape, probs_shape = x.size(), probs.size()
        x = x.view(-1, x.size(-1))
        probs = probs.view(-1)
        assert x.size(0) == probs.size(0), "first dimension of x and probs must be the same"
        assert probs.dtype == torch.float32, "probs must be float32"
        assert act_type in SUPPORTED_ACT_TYPES, f"Unsupported act_type: {act_type}. Supported types: {SUPPORTED_ACT_TYPES}"
        if row_mask is not None:
            assert row_mask.is_cuda, "row_mask must be a CUDA tensor"
            assert x.size(0) == row_mask.size(0), "first dimension of x and row_mask must be the same"
            assert row_mask.ndim == 1, "row_mask must be 1D tensor"
            assert row_mask.dtype == torch.int64, "The dtype of row_mask must be torch.int64."
        out = glu_fwd_with_probs(x, probs, row_mask, act_type)
        ctx.save_for_backward(x, probs, row_mask)
        ctx.act_type, ctx.x_shape, ctx.probs_shape = act_type, x_shape, probs_shape
        return out

    @staticmethod
    def backward(ctx, grad_output):
        assert grad_output.ndim == 2
        x, probs, row_mask = ctx.saved_tensors
        grad_x, grad_probs = glu_bwd_with_probs(grad_output, x, probs, row_mask, ctx.act_type)
        return grad_x.view(ctx.x_shape), grad_probs.view(ctx.probs_shape), None, None


def swiglu_with_probs(x: torch.Tensor, probs: torch.Tensor, row_mask: Union[torch.Tensor, None]) -> torch.Tensor:
    """silu(x[..., :H]) * x[..., H:] * probs -> [tokens, H] (the leading dimensions of x are flattened, as in the reference)."""
    return GLUWithProbs.apply(x, probs, row_mask, "silu")


def geglu_with_probs(x: torch.Tensor, probs: torch.Tensor, row_mask: Union[torch.Tensor, None]) -> torch.Tensor:
    """gelu(x[..., :H]) * x[..., H:] * probs, GELU in its erf form."""
    return GLUWithProbs.apply(x, probs, row_mask, "gelu")
