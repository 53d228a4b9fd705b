"""Float8Linear: torch.nn.Linear whose matmul runs through gemm_fp8.

Same constructor, forward and from_float as the reference's module (primus_turbo/pytorch/modules/linear_fp8.py:20-124);
`cache_quantized_weight` is an addition: the weight is quantized once per optimizer step instead of once per call.
"""
from typing import Optional

import torch

from ..core.low_precision import Float8QuantConfig, ScalingGranularity
from ..ops.gemm_fp8 import gemm_fp8
from ..ops.utils import _get_fp8_dtype
from ._weight_cache import QuantizedWeightCache, needs_transpose_copy

__all__ = ["Float8Linear"]


class Float8Linear(torch.nn.Linear):
    def __init__(self, in_features: int, out_features: int, bias: bool = True, config: Optional[Float8QuantConfig] = None,
                 cache_quantized_weight: bool = False, **kwargs):
        super().__init__(in_features, out_features, bias, **kwargs)
        if config is None:
            config = Float8QuantConfig(granularity=ScalingGranularity.TENSORWISE)
        self.config = config
        self.cache_quantized_weight = cache_quantized_weight

    def _weight_operand(self):
        if not getattr(self, "cache_quantized_weight", False):
            return self.weight
        cache = self.__dict__.get("_qcache")
        if cache is None:
            cache = self.__dict__["_qcache"] = QuantizedWeightCache()
        grad = self.weight.requires_grad and torch.is_grad_enabled()
        return cache.get(self.weight, _get_fp8_dtype(self.config.format, True), self.config,
                         need_transpose=grad and needs_transpose_copy(self.config))

    def clear_quantized_weight_cache(self):
        """Drops the cached quantized weight (needed only after a write that bypasses the parameter's version counter)."""
        cache = self.__dict__.get("_qcache")
        if cache is not None:
            cache.clear()

    def forward(self, x):
        flatten_shapes = x.shape[:-1]
        x_2d = x.reshape(-1, self.in_features)
        out_2d = gemm_fp8(x_2d, self._weight_operand(), trans_a=False, trans_b=True, out_dtype=x.dtype, config=self.config)
        if self.bias is not None:
            out_2d = out_2d + self.bias
        return out_2d.view(*flatten_shapes, self.out_features)

    @classmethod
    @torch.no_grad()
    def from_float(cls, mod: torch.nn.Linear, config: Optional[Float8QuantConfig] = None, inplace: bool = True,
                   cache_quantized_weight: bool = False):
        """Converts a torch.nn.Linear; in place by default (the module object changes class), else into a new module
        with copied parameters."""
        assert isinstance(mod, torch.nn.Linear), f"Expected torch.nn.Linear, got {type(mod)}"
        if config is None:
            config = Float8QuantConfig(granularity=ScalingGranularity.TENSORWISE)
        if inplace:
            mod.__class__ = cls
            mod.config = config
            mod.cache_quantized_weight = cache_quantized_weight
            return mod
        new = cls(mod.in_features, mod.out_features, bias=mod.bias is not None, config=config,
                  cache_quantized_weight=cache_quantized_weight, device=mod.weight.device, dtype=mod.weight.dtype)
        new.weight.copy_(mod.weight)
        if mod.bias is not None:
            new.bias.copy_(mod.bias)
        return new

    def extra_repr(self):
        return f"{super().extra_repr()}, config={getattr(self, 'config', None)}"
