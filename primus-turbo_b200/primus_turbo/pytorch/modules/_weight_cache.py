"""Quantized-weight cache shared by the low-precision linear modules.

A weight is unchanged between optimizer steps, so its quantized copies can be reused by every micro-batch of a
gradient-accumulation window and by every call in inference.  The cache is keyed on the parameter's version counter
(bumped by any in-place update, which is how optimizers write) and storage pointer; the cached QuantizedTensor is tied
back to the parameter with an identity autograd node so that the weight gradient still reaches it.

A write that goes around the version counter is not seen by that key.  The common case is a mixed-precision /
distributed optimizer that keeps fp32 main parameters and copies them into the model with `param.data.copy_(main)`
(the Megatron main_grad flow this package's `fuse_bgrad_accum_pattern="megatron"` serves): `.data` writes never bump
`_version`.  For those flows the key also holds a process-wide generation number: call
`invalidate_quantized_weight_caches()` once per optimizer step, or let `invalidate_on_optimizer_step(optimizer)` do it
from a step post-hook.  A module's `clear_quantized_weight_cache()` drops one cache.
"""
import torch

_generation = 0


def invalidate_quantized_weight_caches() -> None:
    """Makes every quantized-weight cache of the process re-quantize on its next use."""
    global _generation
    _generation += 1


def invalidate_on_optimizer_step(optimizer):
    """Registers a step post-hook on `optimizer` that invalidates all quantized-weight caches; returns the hook handle.
    Needed for optimizers that write the model's parameters through `.data` (main-parameter copies)."""
    return optimizer.register_step_post_hook(lambda *args, **kwargs: invalidate_quantized_weight_caches())

from ..core.quantized_tensor import QuantizedTensor, QuantizedTensorPair, create_quantized_weight


class _TieToParameter(torch.autograd.Function):
    """forward: hands out the cached quantized copy; backward: routes its gradient to the parameter."""

    @staticmethod
    def forward(ctx, weight: torch.Tensor, quantized: QuantizedTensor):
        return quantized.detach()

    @staticmethod
    def backward(ctx, grad):
        return grad, None


class QuantizedWeightCache:
    def __init__(self):
        self._key = None
        self._pair = (None, None)

    def clear(self):
        self._key, self._pair = None, (None, None)

    def get(self, weight: torch.Tensor, dest_dtype: torch.dtype, config, need_transpose: bool) -> QuantizedTensorPair:
        key = (_generation, weight._version, weight.data_ptr(), tuple(weight.shape), weight.dtype, dest_dtype,
               config.granularity, config.block_size, need_transpose)
        if key != self._key:
            self._pair = create_quantized_weight(weight, dest_dtype, config, need_weight_transpose_cache=need_transpose)
            self._key = key
        qw, qw_t = self._pair
        if weight.requires_grad and torch.is_grad_enabled():
            qw = _TieToParameter.apply(weight, qw)
        return QuantizedTensorPair(qw, qw_t)


def needs_transpose_copy(config) -> bool:
    """Whether backward reads a second quantized copy of the weight for this recipe."""
    from ..core.low_precision import Float4QuantConfig, ScalingGranularity
    if isinstance(config, Float4QuantConfig):
        return True
    return config.granularity in (ScalingGranularity.ROWWISE, ScalingGranularity.MX_BLOCKWISE)
