"""Quantized-weight cache shared by the low-precision linear modules.

A weight is unchanged between optimizer steps, so its quantized copies can be reused by every micro-batch of a
gradient-accumulation window and by every call in inference.  The cache is keyed on the parameter's version counter
(bumped by any in-place update, which is how optimizers write) and storage pointer; the cached QuantizedTensor is tied
back to the parameter with an identity autograd node so that the weight gradient still reaches it.

A write that goes around the version counter (`weight.data.add_(...)`, a raw pointer write from another library) is
not seen: call the module's `clear_quantized_weight_cache()` after such an update.
"""
import torch

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
        key = (weight._version, weight.data_ptr(), tuple(weight.shape), weight.dtype, dest_dtype, config.granularity,
               config.block_size, need_transpose)
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
