"""grouped_gemm_fp4: MXFP4 MoE grouped GEMM with autograd
(primus_turbo/pytorch/ops/grouped_gemm_fp4.py:102-400 of the reference)."""
from typing import Optional, Union

import torch

from ..core.low_precision import MXFP4_BLOCK_SIZE, Float4QuantConfig, ScalingGranularity, ScalingRecipe, float4_e2m1fn_x2
from ..core.quantized_tensor import QuantizedTensor, QuantizedTensorPair, check_quantized_tensor
from ..kernels.grouped_gemm.grouped_gemm_fp4_impl import (grouped_gemm_fp4_impl, grouped_gemm_fp4_variable_k_accum_impl,
                                                          grouped_gemm_fp4_variable_k_impl)
from ..kernels.grouped_gemm.grouped_gemm_utils import group_offs_from_lens
from ..kernels.quantization.quantization_impl import grouped_quantize_mxfp4_impl, quantize_mxfp4_impl
from .utils import _get_dummy_wgrad, _setup_fused_grad_accum

__all__ = ["grouped_gemm_fp4"]


class FP4GroupedGemmMXFunc(torch.autograd.Function):
    @staticmethod
    def forward(ctx, a, b, a_t, b_t, group_lens, group_offs, trans_b, out_dtype, config, num_cu, fuse_bgrad_accum_pattern=None):
        fuse, main_grad = _setup_fused_grad_accum(b, fuse_bgrad_accum_pattern)
        assert config.granularity == ScalingGranularity.MX_BLOCKWISE
        assert a.dim() == 2 and b.dim() == 3
        assert out_dtype in (torch.float16, torch.bfloat16)
        assert trans_b, "MXFP4 grouped GEMM only supports trans_b=True (NT layout)."
        N, K = int(b.shape[-2]), int(b.shape[-1])
        assert K % MXFP4_BLOCK_SIZE == 0, f"K must be a multiple of {MXFP4_BLOCK_SIZE} (got {K})."
        assert N % MXFP4_BLOCK_SIZE == 0, f"N must be a multiple of {MXFP4_BLOCK_SIZE} (got {N})."
        total_m = int(a.size(0))
        plain, rht, two_d = ScalingRecipe(), ScalingRecipe(use_rht=True), ScalingRecipe(use_2d_block=True)
        if not isinstance(a, QuantizedTensor):
            a_row, a_row_s, a_col, a_col_s, _, offs_row, _, _ = grouped_quantize_mxfp4_impl(
                a, float4_e2m1fn_x2, None, MXFP4_BLOCK_SIZE, group_lens, group_offs, with_trans=True,
                scaling_recipe=plain, scaling_recipe_for_trans=rht)
        else:
            # pre-quantized row-wise grouped activation; the column-wise (Hadamard-rotated) copy comes from a_t or from
            # re-quantizing the dequantized values (ops/grouped_gemm_fp4.py:156-174 of the reference)
            check_quantized_tensor(a, config, axis=-1, scaling_recipe=plain)
            a_tq = a_t if a_t is not None else QuantizedTensor.quantize(
                a.dequantize(), a.real_dtype, config.granularity, axis=-2, block_size=config.block_size, scaling_recipe=rht,
                group_lens=group_lens)
            a_row, a_row_s, a_col, a_col_s = a.qdata, a.scale_inv, a_tq.qdata, a_tq.scale_inv
            offs_row = a.group_offs
        if not isinstance(b, QuantizedTensor):
            b_row, b_row_s, b_col, b_col_s = quantize_mxfp4_impl(b, float4_e2m1fn_x2, None, MXFP4_BLOCK_SIZE, with_trans=True,
                                                                 scaling_recipe=two_d, scaling_recipe_for_trans=two_d)
        else:
            check_quantized_tensor(b, config, axis=-1, scaling_recipe=two_d)
            b_tq = b_t if b_t is not None else QuantizedTensor.quantize(
                b.dequantize(), b.real_dtype, config.granularity, axis=-2, block_size=config.block_size, scaling_recipe=two_d)
            b_row, b_row_s, b_col, b_col_s = b.qdata, b.scale_inv, b_tq.qdata, b_tq.scale_inv
        out = grouped_gemm_fp4_impl(a_row, b_row, a_row_s, b_row_s, group_lens, offs_row, out_dtype=out_dtype, num_cu=num_cu,
                                    group_offs_out=group_offs)[:total_m]
        ctx.save_for_backward(a_col, a_col_s, b_col, b_col_s, group_lens, group_offs)
        ctx.config, ctx.out_dtype, ctx.num_cu, ctx.total_m, ctx.nk = config, out_dtype, num_cu, total_m, (N, K)
        ctx.fuse, ctx.main_grad = fuse, main_grad
        return out

    @staticmethod
    def backward(ctx, grad_out):
        a_col, a_col_s, b_col, b_col_s, group_lens, group_offs = ctx.saved_tensors
        grad_out = grad_out.contiguous()
        g_row, g_row_s, g_col, g_col_s, _, offs_row, lens_col, offs_col = grouped_quantize_mxfp4_impl(
            grad_out, float4_e2m1fn_x2, None, MXFP4_BLOCK_SIZE, group_lens, group_offs, with_trans=True,
            scaling_recipe=ScalingRecipe(use_sr=ctx.config.use_gradient_sr),
            scaling_recipe_for_trans=ScalingRecipe(use_rht=True, use_sr=ctx.config.use_gradient_sr))
        N, K = ctx.nk
        grad_a = grouped_gemm_fp4_impl(g_row, b_col, g_row_s, b_col_s, group_lens, offs_row, out_dtype=ctx.out_dtype, num_cu=ctx.num_cu,
                                       group_offs_out=group_offs)[:ctx.total_m]
        if ctx.fuse:
            grouped_gemm_fp4_variable_k_accum_impl(g_col, a_col, g_col_s, a_col_s, lens_col, offs_col, ctx.main_grad, num_cu=ctx.num_cu)
            grad_b = _get_dummy_wgrad(ctx.main_grad.shape, ctx.out_dtype, device=ctx.main_grad.device)
        else:
            grad_b = grouped_gemm_fp4_variable_k_impl(g_col, a_col, g_col_s, a_col_s, lens_col, offs_col, ctx.out_dtype, num_cu=ctx.num_cu)
        return (grad_a, grad_b) + (None,) * 9


@torch._dynamo.disable(recursive=True)
def grouped_gemm_fp4(a: Union[torch.Tensor, QuantizedTensor, QuantizedTensorPair], b: Union[torch.Tensor, QuantizedTensor, QuantizedTensorPair],
                     group_lens: torch.Tensor, group_offs: Optional[torch.Tensor] = None, trans_b: bool = True,
                     out_dtype: Optional[torch.dtype] = None, config: Optional[Float4QuantConfig] = None, num_cu: Optional[int] = None,
                     fuse_bgrad_accum_pattern: Optional[str] = None) -> torch.Tensor:
    """out[rows of group g] = a[rows of group g] . b[g]^T with MXFP4 quantization; a [sum(lens), K], b [G, N, K]."""
    if config is None:
        config = Float4QuantConfig()
    if group_offs is None:
        group_offs = group_offs_from_lens(group_lens)
    a_data, a_data_t = (a.data, a.data_t) if isinstance(a, QuantizedTensorPair) else (a, None)
    b_data, b_data_t = (b.data, b.data_t) if isinstance(b, QuantizedTensorPair) else (b, None)
    if out_dtype is None:
        out_dtype = torch.promote_types(a_data.dtype, b_data.dtype)
    return FP4GroupedGemmMXFunc.apply(a_data, b_data, a_data_t, b_data_t, group_lens, group_offs, trans_b, out_dtype, config, num_cu,
                                      fuse_bgrad_accum_pattern)
