"""Grouped (MoE expert) linear layers on the FP8 / FP4 grouped GEMMs.

Shape conventions follow the reference's GroupedLinear (primus_turbo/pytorch/modules/grouped_linear.py:17-52): one
weight [group_num, out_features, in_features], forward(x, group_lens, group_offs) with x [sum(group_lens), in_features]
and group_lens int64 on the device.  The matmul goes through grouped_gemm_fp8 / grouped_gemm_fp4 instead of the bf16
grouped GEMM; `cache_quantized_weight` reuses the quantized experts between optimizer steps.
"""
import math
from typing import Optional

import torch
import torch.nn as nn

from ..core.low_precision import Float4QuantConfig, Float8QuantConfig, ScalingGranularity, float4_e2m1fn_x2
from ..ops.grouped_gemm_fp4 import grouped_gemm_fp4
from ..ops.grouped_gemm_fp8 import grouped_gemm_fp8
from ..ops.utils import _get_fp8_dtype
from ._weight_cache import QuantizedWeightCache, needs_transpose_copy

__all__ = ["Float8GroupedLinear", "Float4GroupedLinear"]


class _LowpGroupedLinear(nn.Module):
    def __init__(self, group_num: int, in_features: int, out_features: int, config, cache_quantized_weight: bool = False,
                 device=None, dtype=None):
        super().__init__()
        self.group_num, self.in_features, self.out_features = group_num, in_features, out_features
        self.config = config
        self.cache_quantized_weight = cache_quantized_weight
        self.weight = nn.Parameter(torch.empty((group_num, out_features, in_features), device=device, dtype=dtype))
        self._qcache = QuantizedWeightCache()
        self.reset_parameters()

    def reset_parameters(self) -> None:
        nn.init.kaiming_uniform_(self.weight, a=math.sqrt(5))

    def _dest_dtype(self):
        raise NotImplementedError

    def _weight_operand(self):
        if not self.cache_quantized_weight:
            return self.weight
        grad = self.weight.requires_grad and torch.is_grad_enabled()
        return self._qcache.get(self.weight, self._dest_dtype(), self.config,
                                need_transpose=grad and needs_transpose_copy(self.config))

    def clear_quantized_weight_cache(self):
        """Drops the cached quantized experts (needed only after a write that bypasses the parameter's version counter)."""
        self._qcache.clear()

    def extra_repr(self) -> str:
        return (f"group_num={self.group_num}, in_features={self.in_features}, out_features={self.out_features}, "
                f"config={self.config}")


class Float8GroupedLinear(_LowpGroupedLinear):
    def __init__(self, group_num: int, in_features: int, out_features: int, config: Optional[Float8QuantConfig] = None,
                 cache_quantized_weight: bool = False, device=None, dtype=None):
        if config is None:
            config = Float8QuantConfig(granularity=ScalingGranularity.TENSORWISE)
        super().__init__(group_num, in_features, out_features, config, cache_quantized_weight, device, dtype)

    def _dest_dtype(self):
        return _get_fp8_dtype(self.config.format, True)

    def forward(self, x: torch.Tensor, group_lens: torch.Tensor, group_offs: Optional[torch.Tensor] = None) -> torch.Tensor:
        return grouped_gemm_fp8(x, self._weight_operand(), group_lens, group_offs, trans_b=True, out_dtype=x.dtype,
                                config=self.config)


class Float4GroupedLinear(_LowpGroupedLinear):
    def __init__(self, group_num: int, in_features: int, out_features: int, config: Optional[Float4QuantConfig] = None,
                 cache_quantized_weight: bool = False, device=None, dtype=None):
        if config is None:
            config = Float4QuantConfig()
        super().__init__(group_num, in_features, out_features, config, cache_quantized_weight, device, dtype)

    def _dest_dtype(self):
        return float4_e2m1fn_x2

    def forward(self, x: torch.Tensor, group_lens: torch.Tensor, group_offs: Optional[torch.Tensor] = None) -> torch.Tensor:
        return grouped_gemm_fp4(x, self._weight_operand(), group_lens, group_offs, trans_b=True, out_dtype=x.dtype,
                                config=self.config)
