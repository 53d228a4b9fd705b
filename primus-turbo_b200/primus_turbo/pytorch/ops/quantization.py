"""Public quantize / dequantize operators.

Signatures and return layouts follow primus_turbo/pytorch/ops/quantization.py of the reference
(quantize_fp8 :52, quantize_fp8_with_trans :103, dequantize_fp8 :225, quantize_fp4 :299,
quantize_fp4_with_trans :446, dequantize_fp4 :486; grouped forms: grouped_quantize_fp8 :144,
grouped_quantize_fp8_with_trans :182, grouped_dequantize_fp8 :272, grouped_quantize_fp4 :340,
grouped_quantize_fp4_with_trans :390, grouped_dequantize_fp4 :519).
"""
from typing import Optional, Tuple

import torch

from ..core.low_precision import MXFP4_BLOCK_SIZE, MXFP8_BLOCK_SIZE, ScalingGranularity, ScalingRecipe
from ..kernels.quantization.quantization_impl import (dequant_fp8_blockwise_for_weight_impl, dequant_fp8_blockwise_impl,
                                                      dequantize_fp8_rowwise_impl, dequantize_fp8_tensorwise_impl,
                                                      dequantize_mxfp4_impl, dequantize_mxfp8_impl,
                                                      grouped_dequantize_mxfp8_impl, grouped_quantize_mxfp4_impl,
                                                      grouped_quantize_mxfp8_impl,
                                                      quant_fp8_blockwise_dual_impl, quant_fp8_blockwise_for_weight_impl,
                                                      quant_fp8_blockwise_impl, quantize_fp8_rowwise_impl,
                                                      quantize_fp8_tensorwise_impl, quantize_mxfp4_impl,
                                                      quantize_mxfp8_impl, shuffle_scale_impl, shuffle_weight_impl)

__all__ = ["quantize_fp8", "quantize_fp8_with_trans", "dequantize_fp8", "quantize_fp4", "quantize_fp4_with_trans",
           "dequantize_fp4", "grouped_quantize_fp8", "grouped_quantize_fp8_with_trans", "grouped_dequantize_fp8",
           "grouped_quantize_fp4", "grouped_quantize_fp4_with_trans", "grouped_dequantize_fp4", "shuffle_scale", "shuffle_weight"]


def shuffle_scale(scale: torch.Tensor, layout=(16, 16)) -> torch.Tensor:
    """ue8m0 scales [M, N] in the pre-shuffled tile order, [ceil(M, 256), ceil(N, 8)], padding 0
    (torch.ops.primus_turbo_cpp_extension.shuffle_scale of the reference)."""
    return shuffle_scale_impl(scale, layout)


def shuffle_weight(weight: torch.Tensor, layout=(16, 16)) -> torch.Tensor:
    """MX codes [M, K] (M % 16 == 0, K % 32 == 0 bytes) in the pre-shuffled tile order, same shape
    (torch.ops.primus_turbo_cpp_extension.shuffle_weight of the reference)."""
    return shuffle_weight_impl(weight, layout)


def _mx_axis(x, axis):
    """Maps negative axes onto the (0, 1) / (1, 2) convention of the MX kernels."""
    if axis is None:
        return None
    return axis if axis >= 0 else x.dim() + axis


def quantize_fp8(x: torch.Tensor, out_dtype: torch.dtype, granularity: ScalingGranularity, *,
                 block_size: Optional[int] = None, axis: Optional[int] = None,
                 scaling_recipe: Optional[ScalingRecipe] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    if granularity == ScalingGranularity.TENSORWISE:
        return quantize_fp8_tensorwise_impl(x, out_dtype)
    if granularity == ScalingGranularity.ROWWISE:
        if axis is None:
            raise ValueError("axis must be specified for rowwise FP8 quantization")
        return quantize_fp8_rowwise_impl(x, out_dtype, axis)
    if granularity == ScalingGranularity.BLOCKWISE:
        assert block_size is not None, "block_size must be specified for BLOCKWISE quantization"
        if scaling_recipe is not None and scaling_recipe.use_2d_block:
            return quant_fp8_blockwise_for_weight_impl(x, out_dtype, block_size=block_size)
        assert axis is not None, "axis must be specified for 1D BLOCKWISE quantization"
        return quant_fp8_blockwise_impl(x, out_dtype, axis=axis, block_size=block_size)
    if granularity == ScalingGranularity.MX_BLOCKWISE:
        assert block_size == MXFP8_BLOCK_SIZE, f"The block size must be {MXFP8_BLOCK_SIZE} for MXFP8 quantization"
        return quantize_mxfp8_impl(x, out_dtype, _mx_axis(x, axis), block_size, False, scaling_recipe)
    raise NotImplementedError(f"Unknown granularity {granularity}")


def quantize_fp8_with_trans(x: torch.Tensor, out_dtype: torch.dtype, granularity: ScalingGranularity, *,
                            block_size: Optional[int] = None, scaling_recipe: Optional[ScalingRecipe] = None,
                            scaling_recipe_for_trans: Optional[ScalingRecipe] = None):
    """Returns (x_rowwise, scale_inv_rowwise, x_colwise, scale_inv_colwise) from one read of x."""
    if granularity == ScalingGranularity.MX_BLOCKWISE:
        assert block_size == MXFP8_BLOCK_SIZE, f"The block size must be {MXFP8_BLOCK_SIZE} for MXFP8 quantization"
        return quantize_mxfp8_impl(x, out_dtype, None, block_size, True, scaling_recipe, scaling_recipe_for_trans)
    if granularity == ScalingGranularity.BLOCKWISE:
        return quant_fp8_blockwise_dual_impl(x, out_dtype, block_size=block_size)
    raise NotImplementedError(f"Unknown granularity {granularity}")


def dequantize_fp8(x: torch.Tensor, out_dtype: torch.dtype, granularity: ScalingGranularity, *,
                   block_size: Optional[int] = None, axis: Optional[int] = None, scale_inv: torch.Tensor,
                   scaling_recipe: Optional[ScalingRecipe] = None):
    if granularity == ScalingGranularity.TENSORWISE:
        return dequantize_fp8_tensorwise_impl(x, out_dtype, scale_inv)
    if granularity == ScalingGranularity.ROWWISE:
        if axis is None:
            raise ValueError("axis must be specified for rowwise FP8 de-quantization")
        return dequantize_fp8_rowwise_impl(x, out_dtype, axis, scale_inv)
    if granularity == ScalingGranularity.BLOCKWISE:
        assert block_size is not None, "block_size must be specified for BLOCKWISE de-quantization"
        if scaling_recipe is not None and scaling_recipe.use_2d_block:
            return dequant_fp8_blockwise_for_weight_impl(x, scale_inv, out_dtype, block_size)
        assert axis is not None, "axis must be specified for 1D BLOCKWISE de-quantization"
        return dequant_fp8_blockwise_impl(x, scale_inv, out_dtype, axis, block_size)
    if granularity == ScalingGranularity.MX_BLOCKWISE:
        assert block_size == MXFP8_BLOCK_SIZE, f"The block size must be {MXFP8_BLOCK_SIZE} for MXFP8 quantization"
        return dequantize_mxfp8_impl(x, out_dtype, _mx_axis(x, axis), block_size, scale_inv)
    raise NotImplementedError(f"Unknown granularity {granularity}")


def quantize_fp4(x: torch.Tensor, out_dtype: torch.dtype, granularity: ScalingGranularity, *,
                 block_size: Optional[int] = None, axis: Optional[int] = None,
                 scaling_recipe: Optional[ScalingRecipe] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    if granularity != ScalingGranularity.MX_BLOCKWISE:
        raise NotImplementedError(f"Unknown granularity {granularity}")
    assert block_size == MXFP4_BLOCK_SIZE, f"The block size must be {MXFP4_BLOCK_SIZE} for MXFP4 quantization"
    return quantize_mxfp4_impl(x, out_dtype, _mx_axis(x, axis), block_size, False, scaling_recipe)


def quantize_fp4_with_trans(x: torch.Tensor, out_dtype: torch.dtype, granularity: ScalingGranularity, *,
                            block_size: Optional[int] = None, scaling_recipe: Optional[ScalingRecipe] = None,
                            scaling_recipe_for_trans: Optional[ScalingRecipe] = None):
    if granularity != ScalingGranularity.MX_BLOCKWISE:
        raise NotImplementedError(f"Unknown granularity {granularity}")
    assert block_size == MXFP4_BLOCK_SIZE, f"The block size must be {MXFP4_BLOCK_SIZE} for MXFP4 quantization"
    return quantize_mxfp4_impl(x, out_dtype, None, block_size, True, scaling_recipe, scaling_recipe_for_trans)


def dequantize_fp4(x: torch.Tensor, out_dtype: torch.dtype, granularity: ScalingGranularity, *,
                   block_size: Optional[int] = None, axis: Optional[int] = None, scale_inv: torch.Tensor,
                   scaling_recipe: Optional[ScalingRecipe] = None):
    if granularity != ScalingGranularity.MX_BLOCKWISE:
        raise NotImplementedError(f"Unknown granularity {granularity}")
    assert block_size == MXFP4_BLOCK_SIZE, f"The block size must be {MXFP4_BLOCK_SIZE} for MXFP4 quantization"
    return dequantize_mxfp4_impl(x, out_dtype, _mx_axis(x, axis), block_size, scale_inv)


# ------------------------------------------------------------------------------ grouped (MoE activations)
def grouped_quantize_fp8(x: torch.Tensor, out_dtype: torch.dtype, granularity: ScalingGranularity, group_lens: torch.Tensor,
                         group_offs: torch.Tensor, *, block_size: Optional[int] = None, axis: Optional[int] = None,
                         scaling_recipe: Optional[ScalingRecipe] = None):
    """x [total_m, N] grouped along M.  Returns (data, scale_inv, group_lens_padded, group_offs_padded): the row-wise
    copy (axis 1, groups padded to 32 rows) or the column-wise, transposed copy (axis 0, groups padded to 128)."""
    if granularity == ScalingGranularity.MX_BLOCKWISE:
        assert block_size == MXFP8_BLOCK_SIZE, f"The block size must be {MXFP8_BLOCK_SIZE} for MXFP8 quantization"
        return grouped_quantize_mxfp8_impl(x, out_dtype, _mx_axis(x, axis), block_size, group_lens, group_offs, False,
                                           scaling_recipe)
    raise NotImplementedError(f"Unknown granularity {granularity}")


def grouped_quantize_fp8_with_trans(x: torch.Tensor, out_dtype: torch.dtype, granularity: ScalingGranularity,
                                    group_lens: torch.Tensor, group_offs: torch.Tensor, *, block_size: Optional[int] = None,
                                    scaling_recipe: Optional[ScalingRecipe] = None,
                                    scaling_recipe_for_trans: Optional[ScalingRecipe] = None):
    """Both copies from one read of x: (x_row, scale_row, x_col, scale_col, group_lens_padded_row,
    group_offs_padded_row, group_lens_padded_col, group_offs_padded_col)."""
    if granularity == ScalingGranularity.MX_BLOCKWISE:
        assert block_size == MXFP8_BLOCK_SIZE, f"The block size must be {MXFP8_BLOCK_SIZE} for MXFP8 quantization"
        return grouped_quantize_mxfp8_impl(x, out_dtype, None, block_size, group_lens, group_offs, True, scaling_recipe,
                                           scaling_recipe_for_trans)
    raise NotImplementedError(f"Unknown granularity {granularity}")


def grouped_dequantize_fp8(x: torch.Tensor, out_dtype: torch.dtype, granularity: ScalingGranularity, group_offs: torch.Tensor,
                           group_offs_padded: torch.Tensor, *, block_size: Optional[int] = None, axis: Optional[int] = None,
                           scale_inv: torch.Tensor, scaling_recipe: Optional[ScalingRecipe] = None,
                           total_M: Optional[int] = None) -> torch.Tensor:
    if granularity == ScalingGranularity.MX_BLOCKWISE:
        assert block_size == MXFP8_BLOCK_SIZE, f"The block size must be {MXFP8_BLOCK_SIZE} for MXFP8 quantization"
        return grouped_dequantize_mxfp8_impl(x, out_dtype, _mx_axis(x, axis), block_size, scale_inv, group_offs,
                                             group_offs_padded, total_M)
    raise NotImplementedError(f"Unknown granularity {granularity}")


def grouped_quantize_fp4(x: torch.Tensor, out_dtype: torch.dtype, granularity: ScalingGranularity, group_lens: torch.Tensor,
                         group_offs: torch.Tensor, *, block_size: Optional[int] = None, axis: Optional[int] = None,
                         scaling_recipe: Optional[ScalingRecipe] = None):
    """As grouped_quantize_fp8 with packed e2m1: the row-wise copy is tight (row i = input row i), the column-wise
    copy pads each group's tokens for the variable-K GEMM."""
    assert out_dtype == torch.float4_e2m1fn_x2, "The out_dtype must be float4_e2m1fn_x2 for MXFP4 quantization"
    if granularity == ScalingGranularity.MX_BLOCKWISE:
        assert block_size == MXFP4_BLOCK_SIZE, f"The block size must be {MXFP4_BLOCK_SIZE} for MXFP4 quantization"
        assert x.ndim == 2, "grouped MXFP4 quantize expects a 2D packed-M tensor"
        axis = _mx_axis(x, axis)
        assert axis in (0, 1), "axis must be 0 (colwise) or 1 (rowwise) for grouped MXFP4"
        return grouped_quantize_mxfp4_impl(x, out_dtype, axis, block_size, group_lens, group_offs, False, scaling_recipe)
    raise NotImplementedError(f"Unknown granularity {granularity}")


def grouped_quantize_fp4_with_trans(x: torch.Tensor, out_dtype: torch.dtype, granularity: ScalingGranularity,
                                    group_lens: torch.Tensor, group_offs: torch.Tensor, *, block_size: Optional[int] = None,
                                    scaling_recipe: Optional[ScalingRecipe] = None,
                                    scaling_recipe_for_trans: Optional[ScalingRecipe] = None):
    assert out_dtype == torch.float4_e2m1fn_x2, "The out_dtype must be float4_e2m1fn_x2 for MXFP4 quantization"
    if granularity == ScalingGranularity.MX_BLOCKWISE:
        assert block_size == MXFP4_BLOCK_SIZE, f"The block size must be {MXFP4_BLOCK_SIZE} for MXFP4 quantization"
        assert x.ndim == 2, "grouped MXFP4 quantize expects a 2D packed-M tensor"
        return grouped_quantize_mxfp4_impl(x, out_dtype, None, block_size, group_lens, group_offs, True, scaling_recipe,
                                           scaling_recipe_for_trans)
    raise NotImplementedError(f"Unknown granularity {granularity}")


def grouped_dequantize_fp4(x: torch.Tensor, out_dtype: torch.dtype, granularity: ScalingGranularity, *,
                           block_size: Optional[int] = None, axis: Optional[int] = None, scale_inv: torch.Tensor,
                           scaling_recipe: Optional[ScalingRecipe] = None) -> torch.Tensor:
    """Row-wise only: the grouped FP4 row copy is tight, so this is the plain dequantizer."""
    if granularity == ScalingGranularity.MX_BLOCKWISE:
        assert block_size == MXFP4_BLOCK_SIZE, f"The block size must be {MXFP4_BLOCK_SIZE} for MXFP4 quantization"
        return dequantize_mxfp4_impl(x, out_dtype, _mx_axis(x, axis), block_size, scale_inv)
    raise NotImplementedError(f"Unknown granularity {granularity}")
