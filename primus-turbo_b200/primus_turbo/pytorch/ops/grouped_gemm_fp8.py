"""grouped_gemm_fp8: MoE grouped GEMM with FP8 quantization and autograd.

Operator surface and data flow follow primus_turbo/pytorch/ops/grouped_gemm_fp8.py of the reference
(grouped_gemm_fp8 :853-966; Functions Block :99-256, Row :259-446, Tensor :449-601, MX :604-840).
"""
from typing import Optional, Union

import torch

from ..core.low_precision import Float8QuantConfig, ScalingGranularity, ScalingRecipe
from ..core.quantized_tensor import QuantizedTensor, QuantizedTensorPair, check_quantized_tensor
from ..kernels.gemm.gemm_fp8_impl import gemm_fp8_impl
from ..kernels.grouped_gemm.grouped_gemm_fp8_impl import (grouped_gemm_fp8_impl, grouped_gemm_fp8_variable_k_accum_impl,
                                                          grouped_gemm_fp8_variable_k_impl)
from ..kernels.grouped_gemm.grouped_gemm_utils import group_offs_from_lens
from ..kernels.quantization.quantization_impl import (grouped_quantize_mxfp8_impl, quant_fp8_blockwise_for_weight_impl,
                                                      quant_fp8_blockwise_segment_m_row_col_impl, quantize_fp8_rowwise_impl,
                                                      quantize_fp8_tensorwise_impl, quantize_mxfp8_impl)
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
        if isinstance(a, QuantizedTensor) or isinstance(b, QuantizedTensor):
            raise NotImplementedError("pre-quantized grouped MX operands are not supported yet")
        fp8_dtype = _get_fp8_dtype(config.format, True)
        bs = config.block_size
        a_row, a_s_row, a_col, a_s_col, _, offs_pad_row, _, _ = grouped_quantize_mxfp8_impl(
            a, fp8_dtype, None, bs, group_lens, group_offs, with_trans=True)
        two_d = ScalingRecipe(use_2d_block=True)
        b_row, b_s_row, b_col, b_s_col = quantize_mxfp8_impl(b, fp8_dtype, None, bs, with_trans=True, scaling_recipe=two_d,
                                                             scaling_recipe_for_trans=two_d)
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


def _per_group_wgrad(a_q, a_s, g_q, g_s, group_lens, out_dtype, gran, trans_b, row_scales):
    """Tensorwise / rowwise wgrad as one dense TN GEMM per group.  Reads group_lens on the host (one sync): the
    variable-K kernel takes 128-padded token segments, which these two granularities do not produce."""
    lens = group_lens.tolist()
    outs, start = [], 0
    for g, n in enumerate(lens):
        sa = a_s[g] if row_scales else a_s
        sg = g_s[g] if row_scales else g_s
        if n == 0:
            shape = (g_q.shape[1], a_q.shape[1]) if trans_b else (a_q.shape[1], g_q.shape[1])
            outs.append(torch.zeros(shape, dtype=out_dtype, device=a_q.device))
        else:
            outs.append(gemm_fp8_impl(a_q[start:start + n], sa, True, g_q[start:start + n], sg, False, out_dtype, trans_b, gran))
        start += n
    return torch.stack(outs)


class FP8GroupedGemmTensorFunc(torch.autograd.Function):
    @staticmethod
    def forward(ctx, a, b, a_t, b_t, group_lens, group_offs, trans_b, out_dtype, config, num_cu, fuse_bgrad_accum_pattern=None):
        assert fuse_bgrad_accum_pattern is None, "fused main_grad accumulation: use BLOCKWISE or MX_BLOCKWISE"
        assert trans_b, "tensorwise grouped GEMM takes b as [G, N, K]"
        fwd = _get_fp8_dtype(config.format, True)
        a_q, a_s = quantize_fp8_tensorwise_impl(a, fwd)
        b_q, b_s = quantize_fp8_tensorwise_impl(b, fwd)
        out = grouped_gemm_fp8_impl(a_q, b_q, a_s, b_s, group_lens, group_offs, False, True, out_dtype, config.granularity, num_cu)
        ctx.save_for_backward(a_q, a_s, b_q, b_s, group_lens, group_offs)
        ctx.config, ctx.out_dtype, ctx.num_cu = config, out_dtype, num_cu
        return out

    @staticmethod
    def backward(ctx, grad_out):
        from ..kernels.quantization.quantization_impl import transpose_2d
        a_q, a_s, b_q, b_s, group_lens, group_offs = ctx.saved_tensors
        gran = ctx.config.granularity
        g_q, g_s = quantize_fp8_tensorwise_impl(grad_out.contiguous(), _get_fp8_dtype(ctx.config.format, False))
        G, N, K = b_q.shape
        b_t_q = torch.stack([transpose_2d(b_q[g]) for g in range(G)])  # [G, K, N]: dgrad contracts over N
        grad_a = grouped_gemm_fp8_impl(g_q, b_t_q, g_s, b_s, group_lens, group_offs, False, True, ctx.out_dtype, gran, ctx.num_cu)
        grad_b = _per_group_wgrad(a_q, a_s, g_q, g_s, group_lens, ctx.out_dtype, gran, True, False)
        return (grad_a, grad_b) + (None,) * 9


class FP8GroupedGemmRowFunc(torch.autograd.Function):
    @staticmethod
    def forward(ctx, a, b, a_t, b_t, group_lens, group_offs, trans_b, out_dtype, config, num_cu, fuse_bgrad_accum_pattern=None):
        assert fuse_bgrad_accum_pattern is None, "fused main_grad accumulation: use BLOCKWISE or MX_BLOCKWISE"
        assert trans_b, "rowwise grouped GEMM takes b as [G, N, K]"
        fwd = _get_fp8_dtype(config.format, True)
        a_q, a_s = quantize_fp8_rowwise_impl(a, fwd, -1)
        b_q, b_s = quantize_fp8_rowwise_impl(b, fwd, -1)                     # [G, N, 1]
        out = grouped_gemm_fp8_impl(a_q, b_q, a_s, b_s, group_lens, group_offs, False, True, out_dtype, config.granularity, num_cu)
        ctx.save_for_backward(a, b, group_lens, group_offs)
        ctx.config, ctx.out_dtype, ctx.num_cu = config, out_dtype, num_cu
        return out

    @staticmethod
    def backward(ctx, grad_out):
        a, b, group_lens, group_offs = ctx.saved_tensors
        gran = ctx.config.granularity
        fwd, gdt = _get_fp8_dtype(ctx.config.format, True), _get_fp8_dtype(ctx.config.format, False)
        grad_out = grad_out.contiguous()
        g_q, g_s = quantize_fp8_rowwise_impl(grad_out, gdt, -1)
        b_t = b.transpose(1, 2).contiguous()                                 # [G, K, N], scaled along N for dgrad
        b_t_q, b_t_s = quantize_fp8_rowwise_impl(b_t, fwd, -1)
        grad_a = grouped_gemm_fp8_impl(g_q, b_t_q, g_s, b_t_s, group_lens, group_offs, False, True, ctx.out_dtype, gran, ctx.num_cu)
        # wgrad: per group, both operands scaled along the token axis
        lens = group_lens.tolist()
        outs, start = [], 0
        for n in lens:
            if n == 0:
                outs.append(torch.zeros(b.shape[1:], dtype=ctx.out_dtype, device=b.device))
            else:
                a_q, a_s = quantize_fp8_rowwise_impl(a[start:start + n].contiguous(), fwd, 0)
                gg_q, gg_s = quantize_fp8_rowwise_impl(grad_out[start:start + n].contiguous(), gdt, 0)
                outs.append(gemm_fp8_impl(a_q, a_s, True, gg_q, gg_s, False, ctx.out_dtype, True, gran))
            start += n
        return (grad_a, torch.stack(outs)) + (None,) * 9


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
