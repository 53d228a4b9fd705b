"""gemm_fp8: FP8 GEMM with autograd for the four scaling granularities.

Operator surface and per-granularity data flow follow primus_turbo/pytorch/ops/gemm_fp8.py of the
reference (gemm_fp8 :728-826; Functions Tensor :96-275, Row :278-426, Block :429-553, MX :556-717):
which operand is quantized along which axis, which copies are saved for backward, and which
format the gradients use (HYBRID = e4m3 forward, e5m2 backward).
"""
from typing import Optional, Union

import torch

from ..core.low_precision import Float8QuantConfig, ScalingGranularity, ScalingRecipe
from ..core.quantized_tensor import QuantizedTensor, QuantizedTensorPair, check_quantized_tensor
from ..kernels.gemm.gemm_fp8_impl import gemm_fp8_accum_impl, gemm_fp8_impl
from ..kernels.quantization.quantization_impl import quantize_mxfp8_impl
from .quantization import quantize_fp8, quantize_fp8_with_trans
from .utils import _get_dummy_wgrad, _get_fp8_dtype, _setup_fused_grad_accum

__all__ = ["gemm_fp8"]


def _bgrad_gemm(a, a_s, trans_a, b, b_s, trans_b, out_dtype, trans_c, granularity, inplace_add_to_out=False, out=None):
    """wgrad GEMM; when asked, accumulates into `out` (main_grad) and returns a placeholder."""
    if not inplace_add_to_out:
        return gemm_fp8_impl(a, a_s, trans_a, b, b_s, trans_b, out_dtype, trans_c, granularity)
    assert out is not None, "out should not be None when inplace_add_to_out is True"
    gemm_fp8_accum_impl(a, a_s, trans_a, b, b_s, trans_b, out, trans_c, granularity)
    return _get_dummy_wgrad(out.shape, out_dtype, device=out.device)


class FP8GemmTensorFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, a, b, a_t, b_t, trans_a, trans_b, out_dtype, config, fuse_bgrad_accum_pattern=None):
        fuse, main_grad = _setup_fused_grad_accum(b, fuse_bgrad_accum_pattern)
        fwd_dtype = _get_fp8_dtype(config.format, True)
        if isinstance(a, QuantizedTensor):
            check_quantized_tensor(a, config)
            qa = a
        else:
            qa = QuantizedTensor.quantize(a, fwd_dtype, config.granularity, axis=-1)
        if isinstance(b, QuantizedTensor):
            check_quantized_tensor(b, config)
            qb = b
        else:
            qb = QuantizedTensor.quantize(b, fwd_dtype, config.granularity, axis=-1)
        out = gemm_fp8_impl(qa.qdata, qa.scale_inv, trans_a, qb.qdata, qb.scale_inv, trans_b, out_dtype, False,
                            config.granularity)
        ctx.save_for_backward(qa.qdata, qa.scale_inv, qb.qdata, qb.scale_inv)
        ctx.trans_a, ctx.trans_b, ctx.out_dtype, ctx.config = trans_a, trans_b, out_dtype, config
        ctx.fuse, ctx.main_grad = fuse, main_grad
        return out

    @staticmethod
    def backward(ctx, grad_out):
        grad_out = grad_out.contiguous()
        a_q, a_s, b_q, b_s = ctx.saved_tensors
        g = QuantizedTensor.quantize(grad_out, _get_fp8_dtype(ctx.config.format, False), ctx.config.granularity, axis=-1)
        gran = ctx.config.granularity
        a_grad = gemm_fp8_impl(g.qdata, g.scale_inv, False, b_q, b_s, not ctx.trans_b, ctx.out_dtype, ctx.trans_a, gran)
        b_grad = _bgrad_gemm(a_q, a_s, not ctx.trans_a, g.qdata, g.scale_inv, False, ctx.out_dtype, ctx.trans_b, gran,
                             inplace_add_to_out=ctx.fuse, out=ctx.main_grad)
        return a_grad, b_grad, None, None, None, None, None, None, None


class FP8GemmRowFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, a, b, a_t, b_t, trans_a, trans_b, out_dtype, config):
        assert trans_a == False, "trans_a has to be False"  # noqa: E712
        fwd_dtype = _get_fp8_dtype(config.format, True)
        gran = config.granularity
        if isinstance(a, QuantizedTensor):
            check_quantized_tensor(a, config, axis=-1)
            qa = a
        else:
            qa = QuantizedTensor.quantize(a, fwd_dtype, gran, axis=-1)
        # the copy scaled along the other axis is derived from the quantized values, as the reference does
        qa_t = a_t if a_t is not None else QuantizedTensor.quantize(qa.dequantize(), qa.real_dtype, gran, axis=-2)
        b_axis = -1 if trans_b else -2
        if isinstance(b, QuantizedTensor):
            check_quantized_tensor(b, config, axis=b_axis)
            qb = b
        else:
            qb = QuantizedTensor.quantize(b, fwd_dtype, gran, axis=b_axis)
        qb_t = b_t if b_t is not None else QuantizedTensor.quantize(qb.dequantize(), qb.real_dtype, gran,
                                                                   axis=-2 if trans_b else -1)
        out = gemm_fp8_impl(qa.qdata, qa.scale_inv, trans_a, qb.qdata, qb.scale_inv, trans_b, out_dtype, False, gran)
        ctx.save_for_backward(qa_t.qdata, qa_t.scale_inv, qb_t.qdata, qb_t.scale_inv)
        ctx.trans_a, ctx.trans_b, ctx.out_dtype, ctx.config = trans_a, trans_b, out_dtype, config
        return out

    @staticmethod
    def backward(ctx, grad_out):
        grad_out = grad_out.contiguous()
        a_t_q, a_t_s, b_t_q, b_t_s = ctx.saved_tensors
        gdt = _get_fp8_dtype(ctx.config.format, False)
        gran = ctx.config.granularity
        g = QuantizedTensor.quantize(grad_out, gdt, gran, axis=-1)
        a_grad = gemm_fp8_impl(g.qdata, g.scale_inv, False, b_t_q, b_t_s, not ctx.trans_b, ctx.out_dtype, ctx.trans_a, gran)
        g_t = QuantizedTensor.quantize(grad_out, gdt, gran, axis=-2)
        b_grad = gemm_fp8_impl(a_t_q, a_t_s, not ctx.trans_a, g_t.qdata, g_t.scale_inv, False, ctx.out_dtype, ctx.trans_b, gran)
        return a_grad, b_grad, None, None, None, None, None, None


class FP8GemmBlockFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, a, b, a_t, b_t, trans_a, trans_b, out_dtype, config):
        assert trans_a == False, "trans_a has to be False"  # noqa: E712
        fwd_dtype = _get_fp8_dtype(config.format, True)
        gran, bs = config.granularity, config.block_size
        if isinstance(a, QuantizedTensor):
            check_quantized_tensor(a, config, axis=-1)
            a_row, a_row_s = a.qdata, a.scale_inv
            if a_t is None:
                a_t = QuantizedTensor.quantize(a.dequantize(), fwd_dtype, gran, axis=-2, block_size=bs)
            a_col, a_col_s = a_t.qdata, a_t.scale_inv
        else:
            a_row, a_row_s, a_col, a_col_s = quantize_fp8_with_trans(a, fwd_dtype, gran, block_size=bs)
        b_recipe = ScalingRecipe(use_2d_block=True)
        if isinstance(b, QuantizedTensor):
            check_quantized_tensor(b, config, scaling_recipe=b_recipe)
            b_q, b_s = b.qdata, b.scale_inv
        else:
            b_q, b_s = quantize_fp8(b, fwd_dtype, gran, block_size=bs, scaling_recipe=b_recipe)
        out = gemm_fp8_impl(a_row, a_row_s, trans_a, b_q, b_s, trans_b, out_dtype, False, gran)
        ctx.save_for_backward(a_col, a_col_s, b_q, b_s)
        ctx.trans_a, ctx.trans_b, ctx.out_dtype, ctx.config = trans_a, trans_b, out_dtype, config
        return out

    @staticmethod
    def backward(ctx, grad_out):
        a_col, a_col_s, b_q, b_s = ctx.saved_tensors
        gdt = _get_fp8_dtype(ctx.config.format, False)
        gran = ctx.config.granularity
        g_row, g_row_s, g_col, g_col_s = quantize_fp8_with_trans(grad_out.contiguous(), gdt, gran,
                                                                 block_size=ctx.config.block_size)
        grad_a = gemm_fp8_impl(g_row, g_row_s, False, b_q, b_s, not ctx.trans_b, ctx.out_dtype, False, gran)
        grad_b = gemm_fp8_impl(a_col, a_col_s, not ctx.trans_a, g_col, g_col_s, False, ctx.out_dtype, ctx.trans_b, gran)
        return grad_a, grad_b, None, None, None, None, None, None


class FP8GemmMXFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, a, b, a_t, b_t, trans_a, trans_b, out_dtype, config, fuse_bgrad_accum_pattern=None):
        assert trans_a == False and trans_b == True, "trans_a has to be False and trans_b has to be True"  # noqa: E712
        fuse, main_grad = _setup_fused_grad_accum(b, fuse_bgrad_accum_pattern)
        fp8_dtype = _get_fp8_dtype(config.format, True)
        gran, bs = config.granularity, config.block_size
        a_recipe = ScalingRecipe()
        if isinstance(a, QuantizedTensor):
            check_quantized_tensor(a, config, axis=-1, scaling_recipe=a_recipe)
            a_row, a_row_s = a.qdata, a.scale_inv
            if a_t is None:
                a_t = QuantizedTensor.quantize(a.dequantize(), a.real_dtype, gran, axis=-2, block_size=bs,
                                               scaling_recipe=a_recipe)
            a_col, a_col_s = a_t.qdata, a_t.scale_inv
        else:
            a_row, a_row_s, a_col, a_col_s = quantize_mxfp8_impl(a, fp8_dtype, None, bs, with_trans=True,
                                                                 scaling_recipe=a_recipe, scaling_recipe_for_trans=a_recipe)
        b_recipe = ScalingRecipe(use_2d_block=True)
        if isinstance(b, QuantizedTensor):
            check_quantized_tensor(b, config, axis=-1, scaling_recipe=b_recipe)
            b_row, b_row_s = b.qdata, b.scale_inv
            if b_t is None:
                b_t = QuantizedTensor.quantize(b.dequantize(), b.real_dtype, gran, axis=-2, block_size=bs,
                                               scaling_recipe=b_recipe)
            b_col, b_col_s = b_t.qdata, b_t.scale_inv
        else:
            b_row, b_row_s, b_col, b_col_s = quantize_mxfp8_impl(b, fp8_dtype, None, bs, with_trans=True,
                                                                 scaling_recipe=b_recipe, scaling_recipe_for_trans=b_recipe)
        out = gemm_fp8_impl(a_row, a_row_s, False, b_row, b_row_s, True, out_dtype, False, gran)
        ctx.save_for_backward(a_col, a_col_s, b_col, b_col_s)
        ctx.out_dtype, ctx.config, ctx.fuse, ctx.main_grad = out_dtype, config, fuse, main_grad
        return out

    @staticmethod
    def backward(ctx, grad_out):
        a_col, a_col_s, b_col, b_col_s = ctx.saved_tensors
        gdt = _get_fp8_dtype(ctx.config.format, False)
        gran = ctx.config.granularity
        grad_out = grad_out.reshape(grad_out.shape[0], -1).contiguous()
        g_row, g_row_s, g_col, g_col_s = quantize_mxfp8_impl(grad_out, gdt, None, ctx.config.block_size, with_trans=True,
                                                             scaling_recipe=ScalingRecipe(),
                                                             scaling_recipe_for_trans=ScalingRecipe())
        grad_a = gemm_fp8_impl(g_row, g_row_s, False, b_col, b_col_s, True, ctx.out_dtype, False, gran)
        grad_b = _bgrad_gemm(g_col, g_col_s, False, a_col, a_col_s, True, ctx.out_dtype, False, gran,
                             inplace_add_to_out=ctx.fuse, out=ctx.main_grad)
        return grad_a, grad_b, None, None, None, None, None, None, None


@torch._dynamo.disable(recursive=True)
def gemm_fp8(a: Union[torch.Tensor, QuantizedTensor, QuantizedTensorPair],
             b: Union[torch.Tensor, QuantizedTensor, QuantizedTensorPair], trans_a: bool = False, trans_b: bool = False,
             out_dtype: Optional[torch.dtype] = None, config: Optional[Float8QuantConfig] = None,
             fuse_bgrad_accum_pattern: Optional[str] = None) -> torch.Tensor:
    """C = op(a) . op(b) with FP8 quantization of both operands in forward and of the gradient in backward.

    a: (M, K) (or (K, M) with trans_a); b: (K, N), or (N, K) with trans_b.  config defaults to
    TENSORWISE / E4M3.  fuse_bgrad_accum_pattern="megatron" adds the weight gradient straight into
    b.main_grad (TENSORWISE and MX_BLOCKWISE only).
    """
    if config is None:
        config = Float8QuantConfig()
    a_data, a_data_t = (a.data, a.data_t) if isinstance(a, QuantizedTensorPair) else (a, None)
    b_data, b_data_t = (b.data, b.data_t) if isinstance(b, QuantizedTensorPair) else (b, None)
    assert a_data.dim() == 2, "Only 2D tensors are supported"
    assert b_data.dim() == 2, "Only 2D tensors are supported"
    if out_dtype is None:
        out_dtype = torch.promote_types(a_data.dtype, b_data.dtype)
    g = config.granularity
    if g == ScalingGranularity.TENSORWISE:
        return FP8GemmTensorFunction.apply(a_data, b_data, a_data_t, b_data_t, trans_a, trans_b, out_dtype, config,
                                           fuse_bgrad_accum_pattern)
    if g == ScalingGranularity.MX_BLOCKWISE:
        return FP8GemmMXFunction.apply(a_data, b_data, a_data_t, b_data_t, trans_a, trans_b, out_dtype, config,
                                       fuse_bgrad_accum_pattern)
    assert fuse_bgrad_accum_pattern is None, f"fuse_bgrad_accum_pattern is not supported for {g}"
    if g == ScalingGranularity.ROWWISE:
        return FP8GemmRowFunction.apply(a_data, b_data, a_data_t, b_data_t, trans_a, trans_b, out_dtype, config)
    if g == ScalingGranularity.BLOCKWISE:
        return FP8GemmBlockFunction.apply(a_data, b_data, a_data_t, b_data_t, trans_a, trans_b, out_dtype, config)
    raise ValueError(f"Unsupported FP8 ScalingGranularity: {g}")
