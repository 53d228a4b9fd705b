"""GroupedLinear: one [group_num, out_features, in_features] weight applied group by group through grouped_gemm
(same module as primus_turbo/pytorch/modules/grouped_linear.py:17-52 of the reference)."""
import math
from typing import Optional

import torch
import torch.nn as nn

from ..ops.grouped_gemm import grouped_gemm

__all__ = ["GroupedLinear"]


class GroupedLinear(nn.Module):
    def __init__(self, group_num: int, in_features: int, out_features: int, device=None, dtype=None):
        super().__init__()
        self.in_features, self.out_features, self.group_num, self.dtype = in_features, out_features, group_num, dtype
        self.weight = nn.Parameter(torch.empty((group_num, out_features, in_features), device=device, dtype=dtype))
        self.reset_parameters()

    def reset_parameters(self) -> None:
        nn.init.kaiming_uniform_(self.weight, a=math.sqrt(5))

    def forward(self, x: torch.Tensor, group_lens: torch.Tensor, group_offs: Optional[torch.Tensor] = None) -> torch.Tensor:
        return grouped_gemm(x, self.weight, group_lens, group_offs, trans_b=True)

    def extra_repr(self) -> str:
        return f"group_num={self.group_num},in_features={self.in_features}, out_features={self.out_features}"
