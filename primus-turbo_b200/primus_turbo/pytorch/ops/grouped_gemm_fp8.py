"""grouped_gemm_fp8: MoE grouped GEMM with FP8 quantization and autograd.

Operator surface and data flow follow primus_turbo/pytorch/ops/grouped_gemm_fp8.py of the reference
(grouped_gemm_fp8 :853-966; Functions Block :99-256, Row :259-446, Tensor :449-601, MX :604-840).
"""
from typing import Optional, Union

import torch

from ..core.low_precision import Float8QuantConfig, ScalingGranularity, ScalingRecipe
from ..core.quantized_tensor import QuantizedTensor, QuantizedTensorPair, check_quantized_tensor
from ..kernels.grouped_gemm.grouped_gemm_fp8_impl import (grouped_gemm_fp8_impl, grouped_gemm_fp8_variable_k_accum_impl,
                                                          grouped_gemm_fp8_variable_k_impl)
from ..kernels.grouped_gemm.grouped_gemm_utils import group_offs_from_lens
from ..kernels.quantization.quantization_impl import (compute_padded_group_offs, grouped_quantize_mxfp8_impl,
                                                      grouped_transpose_pad, quant_fp8_blockwise_for_weight_impl,
                                                      quant_fp8_blockwise_segment_m_row_col_impl, quantize_fp8_rowwise_impl,
                                                      quantize_fp8_tensorwise_impl, quantize_mxfp8_impl, transpose_batched)
from .utils import _get_dummy_wgrad, _get_fp8_dtype, _setup_fused_grad_accum

__all__ = ["grouped_gemm_fp8"]


def _variable_k(a, b, a_s, b_s, lens, offs, trans_a, trans_b, trans_c, out_dtype, gran, num_cu, inplace_add_to_out=False,
                out=None):
    """Grouped wgrad; accumulates into `out` (main_grad) when asked and then returns a placeholder."""
    if not inplace_add_to_out:
        return grouped_gemm_fp8_variable_k_impl(a, b, a_s, b_s, lens, offs, trans_a, trans_b, trans_c, out_dtype, gran, num_cu)
    assert out is not None, "out should not be None when inplace_add_to_out is True"
    grouped_gemm_fp8_variable_k_accum_impl(a, b, a_s, b_s, lens, offs, trans_a, trans_b, trans_c, out, gran, num_cu)
    return _get_dummy_wgrad(out.shape, out_dtype, device=out.device)


class FP8GroupedGemmBlockFunc(torch.autograd.Function):
    """BLOCKWISE: activations 1 x 128 scales (fused row + segment-padded column quantization), weights 128 x 128."""

    @staticmethod
    def forward(ctx, a, b, a_t, b_t, group_lens, group_offs, trans_b, out_dtype, config, num_cu, fuse_bgrad_accum_pattern=None):
        fuse, main_grad = _setup_fused_grad_accum(b, fuse_bgrad_accum_pattern)
        assert config.granularity == ScalingGranularity.BLOCKWISE
        assert config.block_size in [128], "Only block_size 128 is supported currently."
        if isinstance(a, QuantizedTensor):
            raise NotImplementedError("FP8GroupedGemmBlockFunc does not support a pre-quantized activation `a`")
        assert a.dim() == 2, "Input tensor must be 2-dimensional."
        assert b.dim() == 3, "Weight tensor must be 3-dimensional."
        assert group_lens.size(0) == b.size(0), "group_lens size must match b size(0)."
        assert out_dtype in [torch.float16, torch.bfloat16]
        fwd_dtype = _get_fp8_dtype(config.format, True)
        a_row, a_col, a_s_row, a_s_col, _, _ = quant_fp8_blockwise_segment_m_row_col_impl(a, fwd_dtype, config.block_size,
                                                                                          group_lens, group_offs)
        recipe = ScalingRecipe(use_2d_block=True)
        if isinstance(b, QuantizedTensor):
            check_quantized_tensor(b, config, scaling_recipe=recipe)
            b_q, b_s = b.qdata, b.scale_inv
        else:
            b_q, b_s = quant_fp8_blockwise_for_weight_impl(b, fwd_dtype, block_size=config.block_size)
        out = grouped_gemm_fp8_impl(a_row, b_q, a_s_row, b_s, group_lens, group_offs, False, trans_b, out_dtype,
                                    config.granularity, num_cu)
        ctx.save_for_backward(a_col, a_s_col, b_q, b_s, group_lens, group_offs)
        ctx.trans_b, ctx.config, ctx.out_dtype, ctx.num_cu = trans_b, config, out_dtype, num_cu
        ctx.fuse, ctx.main_grad = fuse, main_grad
        return out

    @staticmethod
    def backward(ctx, grad_out):
        grad_out = grad_out.contiguous()
        a_col, a_s_col, b_q, b_s, group_lens, group_offs = ctx.saved_tensors
        gdt = _get_fp8_dtype(ctx.config.format, False)
        gran = ctx.config.granularity
        g_row, g_col, g_s_row, g_s_col, vk_lens, vk_offs = quant_fp8_blockwise_segment_m_row_col_impl(
            grad_out, gdt, ctx.config.block_size, group_lens, group_offs)
        grad_a = grouped_gemm_fp8_impl(g_row, b_q, g_s_row, b_s, group_lens, group_offs, False, not ctx.trans_b, ctx.out_dtype,
                                       gran, ctx.num_cu)
        grad_b = _variable_k(a_col, g_col, a_s_col, g_s_col, vk_lens, vk_offs, True, False, ctx.trans_b, ctx.out_dtype, gran,
                             ctx.num_cu, inplace_add_to_out=ctx.fuse, out=ctx.main_grad)
        return (grad_a, grad_b) + (None,) * 9


class FP8GroupedGemmMXFunc(torch.autograd.Function):
    """MX_BLOCKWISE: grouped dual MX quantization of the activation / gradient, per-expert dual quantization of the weight."""

    @staticmethod
    def forward(ctx, a, b, a_t, b_t, group_lens, group_offs, trans_b, out_dtype, config, num_cu, fuse_bgrad_accum_pattern=None):
        fuse, main_grad = _setup_fused_grad_accum(b, fuse_bgrad_accum_pattern)
        assert config.granularity == ScalingGranularity.MX_BLOCKWISE
        assert a.dim() == 2 and b.dim() == 3
        assert trans_b, "MXFP8 grouped GEMM only supports trans_b=True (NT layout)."
        fp8_dtype = _get_fp8_dtype(config.format, True)
        bs = config.block_size
        one_d, two_d = ScalingRecipe(), ScalingRecipe(use_2d_block=True)
        if not isinstance(a, QuantizedTensor):
            a_row, a_s_row, a_col, a_s_col, _, offs_pad_row, _, _ = grouped_quantize_mxfp8_impl(
                a, fp8_dtype, None, bs, group_lens, group_offs, with_trans=True)
        else:
            # pre-quantized row-wise grouped activation; the column-wise copy comes from a_t or from re-quantizing
            # the dequantized values, as the reference does (ops/grouped_gemm_fp8.py:663-687)
            check_quantized_tensor(a, config, axis=-1, scaling_recipe=one_d)
            assert a.is_grouped_tensor, "A QuantizedTensor input must be a grouped tensor"
            a_tq = a_t if a_t is not None else QuantizedTensor.quantize(
                a.dequantize(), a.real_dtype, config.granularity, axis=-2, block_size=bs, scaling_recipe=one_d,
                group_lens=group_lens)
            a_row, a_s_row, a_col, a_s_col = a.qdata, a.scale_inv, a_tq.qdata, a_tq.scale_inv
            offs_pad_row = a.group_offs
        if not isinstance(b, QuantizedTensor):
            b_row, b_s_row, b_col, b_s_col = quantize_mxfp8_impl(b, fp8_dtype, None, bs, with_trans=True, scaling_recipe=two_d,
                                                                 scaling_recipe_for_trans=two_d)
        else:
            check_quantized_tensor(b, config, axis=-1, scaling_recipe=two_d)
            b_tq = b_t if b_t is not None else QuantizedTensor.quantize(
                b.dequantize(), b.real_dtype, config.granularity, axis=-2, block_size=bs, scaling_recipe=two_d)
            b_row, b_s_row, b_col, b_s_col = b.qdata, b.scale_inv, b_tq.qdata, b_tq.scale_inv
        total_m = int(a.size(0))
        out = grouped_gemm_fp8_impl(a_row, b_row, a_s_row, b_s_row, group_lens, offs_pad_row, False, True, out_dtype,
                                    ScalingGranularity.MX_BLOCKWISE, num_cu, group_offs_out=group_offs)[:total_m]
        ctx.save_for_backward(a_col, a_s_col, b_col, b_s_col, group_lens, group_offs)
        ctx.config, ctx.out_dtype, ctx.num_cu, ctx.total_m = config, out_dtype, num_cu, total_m
        ctx.fuse, ctx.main_grad = fuse, main_grad
        return out

    @staticmethod
    def backward(ctx, grad_out):
        grad_out = grad_out.contiguous()
        a_col, a_s_col, b_col, b_s_col, group_lens, group_offs = ctx.saved_tensors
        gdt = _get_fp8_dtype(ctx.config.format, False)
        g_row, g_s_row, g_col, g_s_col, _, offs_pad_row, lens_pad_col, offs_pad_col = grouped_quantize_mxfp8_impl(
            grad_out, gdt, None, ctx.config.block_size, group_lens, group_offs, with_trans=True)
        gran = ScalingGranularity.MX_BLOCKWISE
        # dgrad: grad_out . b  ==  grad_out_row . b_col^T with b_col [G, K, N_pad] (the transposed copy), NT as forward
        grad_a = grouped_gemm_fp8_impl(g_row, b_col, g_s_row, b_s_col, group_lens, offs_pad_row, False, True, ctx.out_dtype,
                                       gran, ctx.num_cu, group_offs_out=group_offs)[:ctx.total_m]
        # wgrad: grad_b[g] = grad_out_col[:, seg g] . a_col[:, seg g]^T over the 128-padded token segments -> [G, N, K]
        grad_b = _variable_k(g_col, a_col, g_s_col, a_s_col, lens_pad_col, offs_pad_col, False, False, False, ctx.out_dtype,
                             gran, ctx.num_cu, inplace_add_to_out=ctx.fuse, out=ctx.main_grad)
        K = b_col.shape[1]
        N = g_col.shape[0]
        return (grad_a, grad_b[:, :N, :K]) + (None,) * 9


def _token_minor_wgrad(a_q, a_s, g_q, g_s, group_lens, group_offs, trans_b, out_dtype, gran, num_cu, fuse, main_grad):
    """Tensorwise / rowwise wgrad without a host round trip: both token-major FP8 operands are copied to the
    [features, padded tokens] layout (each group's tokens in a zero-filled 128-aligned segment) and contracted by the
    variable-K kernel.  a_q [M, K], g_q [M, N]; scales are scalars (tensorwise) or per column over all tokens
    (rowwise, as the reference quantizes a grouped tensor along axis -2: primus_turbo/pytorch/core/quantized_tensor.py:309-324).
    Returns grad_b as [G, N, K] (trans_b) or [G, K, N]."""
    G = group_lens.numel()
    plens, poffs = compute_padded_group_offs(group_lens, 128)
    a_t = grouped_transpose_pad(a_q, group_offs, poffs)   # [K, T]
    g_t = grouped_transpose_pad(g_q, group_offs, poffs)   # [N, T]
    if gran == ScalingGranularity.ROWWISE:
        a_s = a_s.reshape(1, -1).expand(G, -1).contiguous()
        g_s = g_s.reshape(1, -1).expand(G, -1).contiguous()
    # variable-K computes lhs . rhs^T per segment; trans_c swaps the operands: [G, N, K] = g_t . a_t^T, [G, K, N] the swap
    return _variable_k(g_t, a_t, g_s, a_s, plens, poffs, False, False, not trans_b, out_dtype, gran, num_cu,
                       inplace_add_to_out=fuse, out=main_grad)


class FP8GroupedGemmTensorFunc(torch.autograd.Function):
    """TENSORWISE: one scale per operand.  Follows FP8GroupedGemmTensorFunc of the reference
    (primus_turbo/pytorch/ops/grouped_gemm_fp8.py:449-601)."""

    @staticmethod
    def forward(ctx, a, b, a_t, b_t, group_lens, group_offs, trans_b, out_dtype, config, num_cu, fuse_bgrad_accum_pattern=None):
        fuse, main_grad = _setup_fused_grad_accum(b, fuse_bgrad_accum_pattern)
        assert config.granularity == ScalingGranularity.TENSORWISE
        fwd = _get_fp8_dtype(config.format, True)
        if isinstance(a, QuantizedTensor):
            check_quantized_tensor(a, config)
            a_q, a_s = a.qdata, a.scale_inv
        else:
            a_q, a_s = quantize_fp8_tensorwise_impl(a.contiguous(), fwd)
        if isinstance(b, QuantizedTensor):
            check_quantized_tensor(b, config)
            b_q, b_s = b.qdata, b.scale_inv
        else:
            b_q, b_s = quantize_fp8_tensorwise_impl(b.contiguous(), fwd)
        b_km = b_q if trans_b else transpose_batched(b_q)                    # [G, N, K]
        out = grouped_gemm_fp8_impl(a_q, b_km, a_s, b_s, group_lens, group_offs, False, True, out_dtype, config.granularity, num_cu)
        ctx.save_for_backward(a_q, a_s, b_q, b_s, group_lens, group_offs)
        ctx.trans_b, ctx.config, ctx.out_dtype, ctx.num_cu = trans_b, config, out_dtype, num_cu
        ctx.fuse, ctx.main_grad = fuse, main_grad
        return out

    @staticmethod
    def backward(ctx, grad_out):
        a_q, a_s, b_q, b_s, group_lens, group_offs = ctx.saved_tensors
        gran = ctx.config.granularity
        g_q, g_s = quantize_fp8_tensorwise_impl(grad_out.contiguous(), _get_fp8_dtype(ctx.config.format, False))
        b_nm = transpose_batched(b_q) if ctx.trans_b else b_q                # [G, K, N]: dgrad contracts over N
        grad_a = grouped_gemm_fp8_impl(g_q, b_nm, g_s, b_s, group_lens, group_offs, False, True, ctx.out_dtype, gran, ctx.num_cu)
        grad_b = _token_minor_wgrad(a_q, a_s, g_q, g_s, group_lens, group_offs, ctx.trans_b, ctx.out_dtype, gran, ctx.num_cu,
                                    ctx.fuse, ctx.main_grad)
        return (grad_a, grad_b) + (None,) * 9


class FP8GroupedGemmRowFunc(torch.autograd.Function):
    """ROWWISE: scales along the contraction axis of every GEMM.  Follows FP8GroupedGemmRowFunc of the reference
    (primus_turbo/pytorch/ops/grouped_gemm_fp8.py:259-446): the copies scaled along the other axis, which backward
    needs, are made in forward and saved as FP8, so the high-precision activation is not kept alive."""

    @staticmethod
    def forward(ctx, a, b, a_t, b_t, group_lens, group_offs, trans_b, out_dtype, config, num_cu, fuse_bgrad_accum_pattern=None):
        fuse, main_grad = _setup_fused_grad_accum(b, fuse_bgrad_accum_pattern)
        assert config.granularity == ScalingGranularity.ROWWISE
        fwd = _get_fp8_dtype(config.format, True)
        b_row_axis, b_col_axis = (-1, -2) if trans_b else (-2, -1)
        if isinstance(a, QuantizedTensor):
            check_quantized_tensor(a, config, axis=-1)
            a_q, a_s = a.qdata, a.scale_inv
            a_hp = None if a_t is not None else a.dequantize()
        else:
            a_hp = a.contiguous()
            a_q, a_s = quantize_fp8_rowwise_impl(a_hp, fwd, -1)
        if isinstance(b, QuantizedTensor):
            check_quantized_tensor(b, config, axis=b_row_axis)
            b_q, b_s = b.qdata, b.scale_inv
            b_hp = None if b_t is not None else b.dequantize()
        else:
            b_hp = b.contiguous()
            b_q, b_s = quantize_fp8_rowwise_impl(b_hp, fwd, b_row_axis)      # scales [G, N, 1] or [G, 1, N]
        b_km = b_q if trans_b else transpose_batched(b_q)                    # [G, N, K]
        out = grouped_gemm_fp8_impl(a_q, b_km, a_s, b_s, group_lens, group_offs, False, True, out_dtype, config.granularity, num_cu)
        # copies scaled along the other axis: a per feature over all tokens, b per K
        if a_t is not None:
            a_c_q, a_c_s = a_t.qdata, a_t.scale_inv
        else:
            a_c_q, a_c_s = quantize_fp8_rowwise_impl(a_hp, fwd, -2)          # [M, K], scales [1, K]
        if b_t is not None:
            b_c_q, b_c_s = b_t.qdata, b_t.scale_inv
        else:
            b_c_q, b_c_s = quantize_fp8_rowwise_impl(b_hp, fwd, b_col_axis)  # scales [G, 1, K] or [G, K, 1]
        b_nm = transpose_batched(b_c_q) if trans_b else b_c_q                # [G, K, N]: dgrad contracts over N
        ctx.save_for_backward(a_c_q, a_c_s, b_nm, b_c_s, group_lens, group_offs)
        ctx.trans_b, ctx.config, ctx.out_dtype, ctx.num_cu = trans_b, config, out_dtype, num_cu
        ctx.fuse, ctx.main_grad = fuse, main_grad
        return out

    @staticmethod
    def backward(ctx, grad_out):
        a_c_q, a_c_s, b_nm, b_c_s, group_lens, group_offs = ctx.saved_tensors
        gran = ctx.config.granularity
        gdt = _get_fp8_dtype(ctx.config.format, False)
        grad_out = grad_out.contiguous()
        g_q, g_s = quantize_fp8_rowwise_impl(grad_out, gdt, -1)
        grad_a = grouped_gemm_fp8_impl(g_q, b_nm, g_s, b_c_s, group_lens, group_offs, False, True, ctx.out_dtype, gran, ctx.num_cu)
        g_c_q, g_c_s = quantize_fp8_rowwise_impl(grad_out, gdt, -2)          # [M, N], scales [1, N]
        grad_b = _token_minor_wgrad(a_c_q, a_c_s, g_c_q, g_c_s, group_lens, group_offs, ctx.trans_b, ctx.out_dtype, gran,
                                    ctx.num_cu, ctx.fuse, ctx.main_grad)
        return (grad_a, grad_b) + (None,) * 9


@torch._dynamo.disable(recursive=True)
def grouped_gemm_fp8(a: Union[torch.Tensor, QuantizedTensor, QuantizedTensorPair],
                     b: Union[torch.Tensor, QuantizedTensor, QuantizedTensorPair], group_lens: torch.Tensor,
                     group_offs: Optional[torch.Tensor] = None, trans_b: bool = True, out_dtype: Optional[torch.dtype] = None,
                     config: Optional[Float8QuantConfig] = None, num_cu: Optional[int] = None,
                     fuse_bgrad_accum_pattern: Optional[str] = None) -> torch.Tensor:
    """out[rows of group g] = a[rows of group g] . op(b[g]) with FP8 quantization of both operands.

    a [sum(group_lens), K]; b [G, N, K] (trans_b) or [G, K, N]; group_lens int64 [G] on the device.  num_cu caps the
    number of persistent CTAs.
    """
    if config is None:
        config = Float8QuantConfig()
    if group_offs is None:
        group_offs = group_offs_from_lens(group_lens)
    a_data, a_data_t = (a.data, a.data_t) if isinstance(a, QuantizedTensorPair) else (a, None)
    b_data, b_data_t = (b.data, b.data_t) if isinstance(b, QuantizedTensorPair) else (b, None)
    if out_dtype is None:
        out_dtype = torch.promote_types(a_data.dtype, b_data.dtype)
    fn = {ScalingGranularity.TENSORWISE: FP8GroupedGemmTensorFunc, ScalingGranularity.ROWWISE: FP8GroupedGemmRowFunc,
          ScalingGranularity.BLOCKWISE: FP8GroupedGemmBlockFunc, ScalingGranularity.MX_BLOCKWISE: FP8GroupedGemmMXFunc}.get(
              config.granularity)
    if fn is None:
        raise ValueError(f"Unsupported FP8 ScalingGranularity: {config.granularity}")
    return fn.apply(a_data, b_data, a_data_t, b_data_t, group_lens, group_offs, trans_b, out_dtype, config, num_cu,
                    fuse_bgrad_accum_pattern)
