"""FP8AllToAll: all-to-all of an activation tensor with the payload quantized to FP8 on the wire.

Same call as the reference's FP8AllToAll (primus_turbo/pytorch/dist/fp8_alltoall.py:24-194): `FP8AllToAll.apply(group,
input_, output_split_sizes, input_split_sizes, fwd_quant, bwd_quant, config)`, TENSORWISE / DYNAMIC only, e4m3 forward and
(HYBRID) e5m2 backward, equal or explicit dim-0 splits, bypass for a group of one.  The wire carries one byte per element
plus one scale for the whole group: over NVLink that halves the bytes of the dispatch / combine exchange of an MoE layer.

One deliberate difference.  The reference quantizes every rank's tensor with that rank's own scale and dequantizes what it
receives with the group's MINIMUM scale_inv, which is exact only when all ranks happen to share one amax.  Here the ranks
first agree on the scale (an all-reduce MAX of the local amax: 4 bytes), quantize with it, and dequantize with its inverse,
so every element is scaled and unscaled by the same number.
"""
from typing import List, Tuple, Union

import torch
import torch.distributed as dist

from ..core.low_precision import (Float8QuantConfig, Format, ScalingGranularity, ScalingStrategy, float8_e4m3, float8_e5m2)
from ..kernels.quantization.quantization_impl import dequantize_fp8_tensorwise_impl, quantize_fp8_tensorwise_impl

__all__ = ["FP8AllToAll"]

_QMAX = {float8_e4m3: 448.0, float8_e5m2: 57344.0}


def _exchange(x: torch.Tensor, out_splits, in_splits, group, quant: bool, fp8_dtype):
    orig_dtype = x.dtype
    x = x.contiguous()
    scale_inv = None
    if quant:
        amax = x.abs().amax().float() if x.numel() else torch.zeros((), dtype=torch.float32, device=x.device)
        dist.all_reduce(amax, op=dist.ReduceOp.MAX, group=group)
        scale = _QMAX[fp8_dtype] / torch.clamp(amax, min=1e-12)
        if x.numel():
            x, scale_inv = quantize_fp8_tensorwise_impl(x, fp8_dtype, scale=scale.reshape(1))
        else:
            x, scale_inv = x.to(fp8_dtype), 1.0 / scale
        x = x.view(torch.uint8)
    if out_splits is None:
        out = torch.empty_like(x)
    else:
        out = torch.empty([sum(out_splits)] + list(x.shape[1:]), dtype=x.dtype, device=x.device)
    dist.all_to_all_single(out, x, output_split_sizes=out_splits, input_split_sizes=in_splits, group=group)
    if out.numel() == 0:
        return torch.empty_like(out, dtype=orig_dtype)
    if quant:
        out = dequantize_fp8_tensorwise_impl(out.view(fp8_dtype), orig_dtype, scale_inv.reshape(()))
    return out


class FP8AllToAll(torch.autograd.Function):
    @staticmethod
    def forward(ctx, group, input_: torch.Tensor, output_split_sizes: Union[List, None], input_split_sizes: Union[List, None],
                fwd_quant: bool, bwd_quant: bool, config: Float8QuantConfig) -> torch.Tensor:
        assert group is not None, "group should not be None."
        assert config.strategy == ScalingStrategy.DYNAMIC
        assert config.granularity == ScalingGranularity.TENSORWISE
        if config.format not in (Format.E4M3, Format.HYBRID):
            raise ValueError("FP8AlltoAll only support E4M3 and HYBRID format.")
        ctx.config, ctx.group, ctx.bwd_quant = config, group, bwd_quant
        ctx.output_split_sizes, ctx.input_split_sizes = output_split_sizes, input_split_sizes
        if dist.get_world_size(group=group) == 1:
            return input_
        return _exchange(input_, output_split_sizes, input_split_sizes, group, fwd_quant, float8_e4m3)

    @staticmethod
    def backward(ctx, grad_output: torch.Tensor) -> Tuple[Union[torch.Tensor, None], ...]:
        if dist.get_world_size(group=ctx.group) == 1:
            return None, grad_output, None, None, None, None, None
        bwd_dtype = float8_e4m3 if ctx.config.format == Format.E4M3 else float8_e5m2
        dgrad = _exchange(grad_output, ctx.input_split_sizes, ctx.output_split_sizes, ctx.group, ctx.bwd_quant, bwd_dtype)
        return None, dgrad, None, None, None, None, None
