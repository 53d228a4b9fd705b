"""gemm_fp4: MXFP4 GEMM with autograd (primus_turbo/pytorch/ops/gemm_fp4.py:76-407 of the reference).

Recipes as in the reference: activation row copy plain, its transposed copy with the 16-point Hadamard transform;
weight copies with 2-D (32 x 32) block scales; gradient row copy plain, transposed copy with the Hadamard
transform.  The transform is orthonormal along the contraction of the wgrad GEMM and cancels there.
"""
from typing import Optional, Union

import torch

from ..core.low_precision import Float4QuantConfig, Format, ScalingRecipe
from ..core.quantized_tensor import QuantizedTensor, QuantizedTensorPair, check_quantized_tensor
from ..kernels.gemm.gemm_fp4_impl import gemm_fp4_accum_impl, gemm_fp4_impl
from .quantization import quantize_fp4_with_trans
from .utils import _get_dummy_wgrad, _setup_fused_grad_accum

__all__ = ["gemm_fp4"]


class FP4GemmMXFunction(torch.autograd.Function):
    @staticmethod
    def get_fp4_dtype(format: Format):
        if format == Format.E2M1_X2:
            return torch.float4_e2m1fn_x2
        raise ValueError(f"Unsupported FP4 format: {format}")

    @staticmethod
    def forward(ctx, a, b, a_t, b_t, trans_a, trans_b, out_dtype, config, fuse_bgrad_accum_pattern=None):
        assert trans_a == False and trans_b == True, "MXFP4 GEMM takes the NT layout (trans_a=False, trans_b=True)"  # noqa: E712
        fuse, main_grad = _setup_fused_grad_accum(b, fuse_bgrad_accum_pattern)
        dt = FP4GemmMXFunction.get_fp4_dtype(config.format)
        a_recipe, a_t_recipe = ScalingRecipe(), ScalingRecipe(use_rht=True)
        b_recipe = ScalingRecipe(use_2d_block=True)
        if isinstance(a, QuantizedTensor):
            check_quantized_tensor(a, config, scaling_recipe=a_recipe)
            a_row, a_row_s = a.qdata, a.scale_inv
            if a_t is None:
                a_t = QuantizedTensor.quantize(a.dequantize(), a.real_dtype, config.granularity, axis=-2,
                                               block_size=config.block_size, scaling_recipe=a_t_recipe)
            a_col, a_col_s = a_t.qdata, a_t.scale_inv
        else:
            a_row, a_row_s, a_col, a_col_s = quantize_fp4_with_trans(a, dt, config.granularity, block_size=config.block_size,
                                                                     scaling_recipe=a_recipe, scaling_recipe_for_trans=a_t_recipe)
        if isinstance(b, QuantizedTensor):
            check_quantized_tensor(b, config, scaling_recipe=b_recipe)
            b_row, b_row_s = b.qdata, b.scale_inv
            if b_t is None:
                b_t = QuantizedTensor.quantize(b.dequantize(), b.real_dtype, config.granularity, axis=-2,
                                               block_size=config.block_size, scaling_recipe=b_recipe)
            b_col, b_col_s = b_t.qdata, b_t.scale_inv
        else:
            b_row, b_row_s, b_col, b_col_s = quantize_fp4_with_trans(b, dt, config.granularity, block_size=config.block_size,
                                                                     scaling_recipe=b_recipe, scaling_recipe_for_trans=b_recipe)
        out = gemm_fp4_impl(a_row, a_row_s, False, b_row, b_row_s, True, out_dtype, False)
        ctx.save_for_backward(a_col, a_col_s, b_col, b_col_s)
        ctx.out_dtype, ctx.config, ctx.fuse, ctx.main_grad = out_dtype, config, fuse, main_grad
        return out

    @staticmethod
    def backward(ctx, grad_out):
        a_col, a_col_s, b_col, b_col_s = ctx.saved_tensors
        dt = FP4GemmMXFunction.get_fp4_dtype(ctx.config.format)
        grad_out = grad_out.reshape(grad_out.shape[0], -1).contiguous()
        g_row, g_row_s, g_col, g_col_s = quantize_fp4_with_trans(grad_out, dt, ctx.config.granularity,
                                                                 block_size=ctx.config.block_size,
                                                                 scaling_recipe=ScalingRecipe(use_sr=ctx.config.use_gradient_sr),
                                                                 scaling_recipe_for_trans=ScalingRecipe(use_rht=True, use_sr=ctx.config.use_gradient_sr))
        grad_a = gemm_fp4_impl(g_row, g_row_s, False, b_col, b_col_s, True, ctx.out_dtype, False)
        if ctx.fuse:
            gemm_fp4_accum_impl(g_col, g_col_s, False, a_col, a_col_s, True, ctx.main_grad, False)
            grad_b = _get_dummy_wgrad(ctx.main_grad.shape, ctx.out_dtype, device=ctx.main_grad.device)
        else:
            grad_b = gemm_fp4_impl(g_col, g_col_s, False, a_col, a_col_s, True, ctx.out_dtype, False)
        return grad_a, grad_b, None, None, None, None, None, None, None


@torch._dynamo.disable(recursive=True)
def gemm_fp4(a: Union[torch.Tensor, QuantizedTensor, QuantizedTensorPair], b: Union[torch.Tensor, QuantizedTensor, QuantizedTensorPair],
             trans_a: bool = False, trans_b: bool = False, out_dtype: Optional[torch.dtype] = None,
             config: Optional[Float4QuantConfig] = None, fuse_bgrad_accum_pattern: Optional[str] = None) -> torch.Tensor:
    """C = a . b^T with MXFP4 quantization (NT layout: a [M, K], b [N, K] with trans_b=True; K, N multiples of 32)."""
    if config is None:
        config = Float4QuantConfig()
    a_data, a_data_t = (a.data, a.data_t) if isinstance(a, QuantizedTensorPair) else (a, None)
    b_data, b_data_t = (b.data, b.data_t) if isinstance(b, QuantizedTensorPair) else (b, None)
    assert a_data.dim() == 2 and b_data.dim() == 2, "Only 2D tensors are supported"
    if out_dtype is None:
        out_dtype = torch.promote_types(a_data.dtype, b_data.dtype)
    return FP4GemmMXFunction.apply(a_data, b_data, a_data_t, b_data_t, trans_a, trans_b, out_dtype, config, fuse_bgrad_accum_pattern)
