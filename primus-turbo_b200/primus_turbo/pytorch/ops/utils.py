"""Helpers shared by the GEMM operators (primus_turbo/pytorch/ops/utils.py:20-89 of the reference)."""
from typing import Optional

import torch

from ..core.low_precision import Format, float8_e4m3, float8_e5m2


def _get_fp8_dtype(format: Format, is_fwd_stage: bool):
    if format == Format.E4M3:
        return float8_e4m3
    if format == Format.E5M2:
        return float8_e5m2
    if format == Format.HYBRID:
        return float8_e4m3 if is_fwd_stage else float8_e5m2
    raise ValueError(f"Unsupported FP8 format: {format}")


def _setup_fused_grad_accum(b, fuse_bgrad_accum_pattern: Optional[str]):
    """Megatron's main_grad convention: returns (enabled, main_grad) and marks the weight so the
    framework skips its own accumulation; the wgrad GEMM then adds straight into main_grad."""
    if fuse_bgrad_accum_pattern is None:
        return False, None
    assert fuse_bgrad_accum_pattern in ["megatron"], "Only megatron support gradient accumulation fusion currently"
    assert hasattr(b, "grad_added_to_main_grad"), "b.grad_added_to_main_grad must be set up before the backward pass."
    assert hasattr(b, "main_grad"), "b.main_grad must be set up before the backward pass."
    assert isinstance(b.main_grad, torch.Tensor) and (b.main_grad.shape == b.shape), \
        "b.main_grad must be a tensor with the same shape as b"
    b.grad_added_to_main_grad = True
    return True, b.main_grad


_dummy_wgrads = {}


def _get_dummy_wgrad(shape, dtype, zero=False, device="cuda"):
    """Cached placeholder returned as the weight gradient when the real one was accumulated in place;
    its contents are never read."""
    key = (tuple(shape), dtype, str(device))
    if key not in _dummy_wgrads:
        _dummy_wgrads[key] = torch.empty(shape, dtype=dtype, device=device, requires_grad=False)
    if zero:
        _dummy_wgrads[key].fill_(0)
    return _dummy_wgrads[key].detach()
