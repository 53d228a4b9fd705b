"""Quantize / dequantize entry points over the C ABI.

Function names, arguments and return layouts follow
primus_turbo/pytorch/kernels/quantization/quantization_impl.py of the reference; each call lands in
one extern "C" function of libpt_b200.so.
"""
from typing import Optional, Tuple

import torch

from ...core.low_precision import ScalingRecipe
from .. import _native as nv

BLOCK = 128
MX_BLOCK = 32
MX_ALIGN = 128


def ceil_div(a, b):
    return (a + b - 1) // b


def _ws(device):
    return torch.empty(64, dtype=torch.int32, device=device)


# ------------------------------------------------------------------------------ tensorwise / rowwise
def quantize_fp8_tensorwise_impl(x: torch.Tensor, out_dtype: torch.dtype,
                                 scale: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    nv.require_cuda(x, scale)
    x = x.contiguous()
    q = torch.empty_like(x, dtype=out_dtype)
    scale_inv = torch.empty((), dtype=torch.float32, device=x.device)
    ws = _ws(x.device)
    if scale is not None:
        assert scale.numel() == 1, "tensorwise scale must be scalar tensor"
        scale = scale.to(torch.float32).contiguous()
    with nv.on_device(x.device):
        nv.check(nv.lib().pt_quantize_fp8_tensorwise(nv.ptr(x), nv.src_code(x.dtype), x.numel(), nv.fmt_code(out_dtype),
                                                      nv.ptr(q), nv.ptr(scale_inv), nv.ptr(scale), nv.ptr(ws),
                                                      ws.numel() * 4, nv.stream(x.device)), "quantize_fp8_tensorwise")
    return q, scale_inv


def quantize_fp8_rowwise_impl(x: torch.Tensor, out_dtype: torch.dtype, axis: int,
                              scale: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    nv.require_cuda(x, scale)
    assert x.is_contiguous(), "The x tensor must be contiguous."
    axis = axis if axis >= 0 else x.dim() + axis
    assert 0 <= axis < x.dim()
    shape = list(x.shape)
    scale_shape = list(shape)
    scale_shape[axis] = 1
    q = torch.empty_like(x, dtype=out_dtype)
    scale_inv = torch.empty(scale_shape, dtype=torch.float32, device=x.device)
    last = axis == x.dim() - 1
    if last:
        B, M, N = 1, x.numel() // max(shape[axis], 1), shape[axis]
    else:
        B = 1
        for s in shape[:axis]:
            B *= s
        M = shape[axis]
        N = 1
        for s in shape[axis + 1:]:
            N *= s
    ws = None
    if not last and scale is None:
        ws = torch.empty(max(B * N, 1), dtype=torch.int32, device=x.device)
    if scale is not None:
        assert list(scale.shape) == scale_shape
        scale = scale.to(torch.float32).contiguous()
    with nv.on_device(x.device):
        nv.check(nv.lib().pt_quantize_fp8_rowwise(nv.ptr(x), nv.src_code(x.dtype), B, M, N, int(last),
                                                   nv.fmt_code(out_dtype), nv.ptr(q), nv.ptr(scale_inv), nv.ptr(scale),
                                                   nv.ptr(ws), 0 if ws is None else ws.numel() * 4,
                                                   nv.stream(x.device)), "quantize_fp8_rowwise")
    return q, scale_inv


def dequantize_fp8_tensorwise_impl(x: torch.Tensor, out_dtype: torch.dtype, scale_inv: torch.Tensor):
    nv.require_cuda(x, scale_inv)
    x = x.contiguous()
    y = torch.empty_like(x, dtype=out_dtype)
    with nv.on_device(x.device):
        nv.check(nv.lib().pt_dequantize_fp8(nv.ptr(x), nv.fmt_code(x.dtype), nv.ptr(scale_inv.contiguous()), 0, 1, 1,
                                             x.numel(), nv.ptr(y), nv.src_code(out_dtype), nv.stream(x.device)),
                 "dequantize_fp8_tensorwise")
    return y


def dequantize_fp8_rowwise_impl(x: torch.Tensor, out_dtype: torch.dtype, axis: int, scale_inv: torch.Tensor):
    nv.require_cuda(x, scale_inv)
    assert x.is_contiguous(), "The x tensor must be contiguous."
    assert scale_inv.is_contiguous(), "The scale_inv tensor must be contiguous."
    axis = axis if axis >= 0 else x.dim() + axis
    shape = list(x.shape)
    y = torch.empty_like(x, dtype=out_dtype)
    if axis == x.dim() - 1:
        kind, B, M, N = 1, 1, x.numel() // max(shape[axis], 1), shape[axis]
    else:
        kind, B = 2, 1
        for s in shape[:axis]:
            B *= s
        M, N = shape[axis], 1
        for s in shape[axis + 1:]:
            N *= s
    with nv.on_device(x.device):
        nv.check(nv.lib().pt_dequantize_fp8(nv.ptr(x), nv.fmt_code(x.dtype), nv.ptr(scale_inv), kind, B, M, N,
                                             nv.ptr(y), nv.src_code(out_dtype), nv.stream(x.device)),
                 "dequantize_fp8_rowwise")
    return y


# ------------------------------------------------------------------------------ 128-blockwise
def quant_fp8_blockwise_impl(x: torch.Tensor, dtype: torch.dtype, axis: int,
                             block_size: int = 128) -> Tuple[torch.Tensor, torch.Tensor]:
    nv.require_cuda(x)
    assert x.is_contiguous() and x.dim() == 2, "Input must be 2D and contiguous"
    assert axis in (-2, -1, 0, 1), f"axis must be 0 or 1 (or -1, -2), got {axis}"
    assert block_size == BLOCK, "block_size must be 128"
    axis = axis % 2
    M, N = x.shape
    q = torch.empty((M, N), dtype=dtype, device=x.device)
    s = torch.empty((M, ceil_div(N, BLOCK)) if axis == 1 else (ceil_div(M, BLOCK), N), dtype=torch.float32,
                    device=x.device)
    args = (nv.ptr(q), nv.ptr(s), None, None) if axis == 1 else (None, None, nv.ptr(q), nv.ptr(s))
    with nv.on_device(x.device):
        nv.check(nv.lib().pt_quantize_fp8_blockwise(nv.ptr(x), nv.src_code(x.dtype), M, N, nv.fmt_code(dtype), *args,
                                                     nv.stream(x.device)), "quant_fp8_blockwise")
    return q, s


def quant_fp8_blockwise_dual_impl(x: torch.Tensor, dtype: torch.dtype, block_size: int = 128):
    """(q_row, s_row [M, N/128], q_col [M, N] not transposed, s_col [M/128, N]) from one read of x."""
    nv.require_cuda(x)
    assert x.is_contiguous() and x.dim() == 2, "Input must be 2D and contiguous"
    assert block_size == BLOCK, "block_size must be 128"
    M, N = x.shape
    q_row = torch.empty((M, N), dtype=dtype, device=x.device)
    q_col = torch.empty((M, N), dtype=dtype, device=x.device)
    s_row = torch.empty((M, ceil_div(N, BLOCK)), dtype=torch.float32, device=x.device)
    s_col = torch.empty((ceil_div(M, BLOCK), N), dtype=torch.float32, device=x.device)
    with nv.on_device(x.device):
        nv.check(nv.lib().pt_quantize_fp8_blockwise(nv.ptr(x), nv.src_code(x.dtype), M, N, nv.fmt_code(dtype),
                                                     nv.ptr(q_row), nv.ptr(s_row), nv.ptr(q_col), nv.ptr(s_col),
                                                     nv.stream(x.device)), "quant_fp8_blockwise_dual")
    return q_row, s_row, q_col, s_col


def quant_fp8_blockwise_for_weight_impl(w: torch.Tensor, dtype: torch.dtype, block_size: int = 128):
    nv.require_cuda(w)
    assert w.dim() in (2, 3), "Weight must be 2D or 3D"
    assert block_size == BLOCK, "block_size must be 128"
    w = w.contiguous()
    B = 1 if w.dim() == 2 else w.shape[0]
    M, N = w.shape[-2:]
    q = torch.empty_like(w, dtype=dtype)
    sshape = (ceil_div(M, BLOCK), ceil_div(N, BLOCK))
    s = torch.empty(sshape if w.dim() == 2 else (B,) + sshape, dtype=torch.float32, device=w.device)
    with nv.on_device(w.device):
        nv.check(nv.lib().pt_quantize_fp8_blockwise_weight(nv.ptr(w), nv.src_code(w.dtype), B, M, N, nv.fmt_code(dtype),
                                                            nv.ptr(q), nv.ptr(s), nv.stream(w.device)),
                 "quant_fp8_blockwise_for_weight")
    return q, s


def compute_padded_group_offs(group_lens: torch.Tensor, align: int):
    nv.require_cuda(group_lens)
    G = group_lens.numel()
    lens = group_lens.to(torch.int64).contiguous()
    plens = torch.empty(G, dtype=torch.int64, device=lens.device)
    poffs = torch.empty(G + 1, dtype=torch.int64, device=lens.device)
    with nv.on_device(lens.device):
        nv.check(nv.lib().pt_compute_padded_group_offs(nv.ptr(lens), G, align, nv.ptr(plens), nv.ptr(poffs),
                                                        nv.stream(lens.device)), "compute_padded_group_offs")
    return plens, poffs


def quant_fp8_blockwise_segment_m_row_col_impl(x: torch.Tensor, dtype: torch.dtype, block_size: int,
                                               group_lens: torch.Tensor, group_offs: torch.Tensor,
                                               gemm_other_dim: Optional[int] = None):
    """Returns (x_row, x_col_padded, scales_row [N/128, M], scales_col_padded, padded_lens, padded_offs)."""
    nv.require_cuda(x, group_lens, group_offs)
    assert x.is_contiguous() and x.dim() == 2, "Input must be 2D and contiguous"
    assert block_size == BLOCK, "block_size must be 128"
    M, N = x.shape
    G = group_lens.numel()
    plens, poffs = compute_padded_group_offs(group_lens, BLOCK)
    m_alloc = M + G * BLOCK
    x_row = torch.empty((M, N), dtype=dtype, device=x.device)
    x_col = torch.empty((m_alloc, N), dtype=dtype, device=x.device)
    s_row = torch.empty((ceil_div(N, BLOCK), M), dtype=torch.float32, device=x.device)
    s_col = torch.empty((m_alloc // BLOCK, N), dtype=torch.float32, device=x.device)
    with nv.on_device(x.device):
        nv.check(nv.lib().pt_quantize_fp8_blockwise_segment_m(
            nv.ptr(x), nv.src_code(x.dtype), M, N, G, nv.ptr(group_offs.to(torch.int64).contiguous()), nv.ptr(poffs),
            nv.fmt_code(dtype), nv.ptr(x_row), nv.ptr(s_row), nv.ptr(x_col), nv.ptr(s_col), nv.stream(x.device)),
            "quant_fp8_blockwise_segment_m_row_col")
    return x_row, x_col, s_row, s_col, plens, poffs


def _dequant_blockwise(x, scales, out_dtype, kind):
    nv.require_cuda(x, scales)
    x = x.contiguous()
    B = 1 if x.dim() == 2 else x.shape[0]
    M, N = x.shape[-2:]
    y = torch.empty_like(x, dtype=out_dtype)
    with nv.on_device(x.device):
        nv.check(nv.lib().pt_dequantize_fp8_blockwise(nv.ptr(x), nv.fmt_code(x.dtype), nv.ptr(scales.contiguous()), kind,
                                                       B, M, N, nv.ptr(y), nv.src_code(out_dtype), nv.stream(x.device)),
                 "dequant_fp8_blockwise")
    return y


def dequant_fp8_blockwise_impl(x: torch.Tensor, scales: torch.Tensor, out_dtype: torch.dtype, axis: int,
                               block_size: int = 128):
    assert block_size == BLOCK
    return _dequant_blockwise(x, scales, out_dtype, 0 if axis % 2 == 1 else 1)


def dequant_fp8_blockwise_for_weight_impl(x: torch.Tensor, scales: torch.Tensor, out_dtype: torch.dtype,
                                          block_size: int = 128):
    assert block_size == BLOCK
    return _dequant_blockwise(x, scales, out_dtype, 2)


# ------------------------------------------------------------------------------ MX
def _launch_fused_mx(pro, x, M, N, fmt, flags, q_row, s_row, q_col, s_col, grouped=None):
    """pro = ("glu", probs, row_mask, act_code) or ("rmsnorm", rstd, gamma, zero_centered): the quantizer applies the
    operator to each tile of x as it loads it.  grouped = (G, offs, poffs_row, poffs_col, col_alloc) for the grouped form."""
    lib, st = nv.lib(), nv.stream(x.device)
    if pro[0] == "glu":
        _, probs, row_mask, act = pro
        if grouped is None:
            nv.check(lib.pt_glu_quantize_mx(nv.ptr(x), nv.src_code(x.dtype), nv.ptr(probs), nv.ptr(row_mask), M, N, act, fmt, flags, nv.ptr(q_row),
                                            nv.ptr(s_row), nv.ptr(q_col), nv.ptr(s_col), st), "glu_quantize_mx")
        else:
            G, offs, poffs_row, poffs_col, col_alloc = grouped
            nv.check(lib.pt_grouped_glu_quantize_mx(nv.ptr(x), nv.src_code(x.dtype), nv.ptr(probs), nv.ptr(row_mask), M, N, act, G, nv.ptr(offs),
                                                    nv.ptr(poffs_row), nv.ptr(poffs_col), fmt, flags, nv.ptr(q_row), nv.ptr(s_row), nv.ptr(q_col),
                                                    nv.ptr(s_col), col_alloc, st), "grouped_glu_quantize_mx")
    else:
        _, rstd, gamma, zero_centered = pro
        assert grouped is None
        nv.check(lib.pt_rmsnorm_quantize_mx(nv.ptr(x), nv.src_code(x.dtype), nv.ptr(rstd), nv.ptr(gamma), int(bool(zero_centered)), M, N, fmt, flags,
                                            nv.ptr(q_row), nv.ptr(s_row), nv.ptr(q_col), nv.ptr(s_col), st), "rmsnorm_quantize_mx")


def fused_mx_supported(x: torch.Tensor, width: int, out_dtype, gated: bool) -> bool:
    """Whether the one-pass kernels take this call: bf16 input, e4m3 or e2m1 codes, 16-byte aligned rows, and for the gated
    activations a width that is a multiple of the 64-column tile.  Outside that the caller runs operator + quantizer."""
    return (x.dtype == torch.bfloat16 and nv.fmt_code(out_dtype) in (nv.PT_E4M3, nv.PT_E2M1) and width % (64 if gated else 32) == 0
            and x.data_ptr() % 16 == 0 and 0 < x.shape[0] < 2 ** 31)


def shuffle_scale_impl(scale: torch.Tensor, layout=(16, 16)) -> torch.Tensor:
    """ue8m0 scale [M, N] -> [ceil(M, 256), ceil(N, 8)] in the pre-shuffled tile order (zero padding).  Mirrors
    torch.ops.primus_turbo_cpp_extension.shuffle_scale of the reference (csrc/pytorch/shuffle/shuffle.cpp:16-50)."""
    nv.require_cuda(scale)
    assert tuple(layout) == (16, 16), "Unsupported shuffle layout."
    assert scale.dim() == 2, "Scale must be 2D"
    assert scale.dtype in (torch.float8_e8m0fnu, torch.uint8), "Scale must be Float8_e8m0fnu."
    src = scale.contiguous().view(torch.uint8)
    M, N = src.shape
    out = torch.empty(ceil_div(M, 256) * 256, ceil_div(N, 8) * 8, dtype=torch.uint8, device=scale.device)
    with nv.on_device(scale.device):
        nv.check(nv.lib().pt_shuffle_e8m0_scale(nv.ptr(src), M, N, nv.ptr(out), nv.stream(scale.device)), "shuffle_scale")
    return out.view(torch.float8_e8m0fnu)


def shuffle_weight_impl(weight: torch.Tensor, layout=(16, 16)) -> torch.Tensor:
    """MXFP4 (packed pairs) or MXFP8 codes [M, K] -> the same shape in the pre-shuffled (16 rows x 32 bytes) tile order.
    Mirrors torch.ops.primus_turbo_cpp_extension.shuffle_weight of the reference (csrc/pytorch/shuffle/shuffle.cpp:52-92),
    which takes MXFP4; the MX quantizers' shuffle_out option uses the same order for FP8 codes."""
    nv.require_cuda(weight)
    assert tuple(layout) == (16, 16), "Unsupported shuffle layout."
    assert weight.dim() == 2, "Weight must be 2D"
    assert weight.is_contiguous(), "Weight must be contiguous"
    src = weight.view(torch.uint8)
    M, K = src.shape
    assert M % 16 == 0, f"M must be divisible by 16 for shuffled codes. But got M={M}"
    assert K % 32 == 0, f"N must be divisible by 32 for shuffled codes. But got N={K}"
    out = torch.empty_like(src)
    with nv.on_device(weight.device):
        nv.check(nv.lib().pt_shuffle_mx_codes(nv.ptr(src), M, K, nv.ptr(out), nv.stream(weight.device)), "shuffle_weight")
    return out.view(weight.dtype)


def _shuffled(q, s, recipe):
    """The shuffle_scale / shuffle_out options of a ScalingRecipe, applied to one copy (2-D, or batched group by group)."""
    if q is None or recipe is None or not (recipe.shuffle_scale or recipe.shuffle_out):
        return q, s
    if recipe.shuffle_scale:
        s = shuffle_scale_impl(s) if s.dim() == 2 else torch.stack([shuffle_scale_impl(t) for t in s])
    if recipe.shuffle_out:
        q = shuffle_weight_impl(q) if q.dim() == 2 else torch.stack([shuffle_weight_impl(t.contiguous()) for t in q])
    return q, s


def _mx_quant(x, out_dtype, want_row, want_col, row_recipe, col_recipe, pro=None):
    nv.require_cuda(x)
    x = x.contiguous()
    fmt = nv.fmt_code(out_dtype)
    fp4 = fmt == nv.PT_E2M1
    for r in (row_recipe, col_recipe):
        if r is not None and r.use_sr and not fp4:
            raise ValueError("stochastic rounding is an MXFP4 option (ScalingRecipe.use_sr)")
    G = 1 if x.dim() == 2 else x.shape[0]
    M, N = x.shape[-2:]
    if pro is not None and pro[0] == "glu":
        N //= 2   # the quantized tensor is act(x[:, :N]) * x[:, N:] * probs
    M_pad, N_pad = ceil_div(M, MX_ALIGN) * MX_ALIGN, ceil_div(N, MX_ALIGN) * MX_ALIGN
    lead = () if x.dim() == 2 else (G,)
    div = 2 if fp4 else 1
    flags = 0
    q_row = s_row = q_col = s_col = None
    if want_row:
        flags |= nv.PT_MX_ROW | (nv.PT_MX_ROW_2D if row_recipe.use_2d_block else 0) | (nv.PT_MX_ROW_RHT if row_recipe.use_rht else 0)
        flags |= nv.PT_MX_ROW_SR if row_recipe.use_sr else 0
        q_row = torch.empty(lead + (M, N_pad // div), dtype=torch.uint8, device=x.device)
        s_row = torch.empty(lead + (M, N_pad // MX_BLOCK), dtype=torch.uint8, device=x.device)
    if want_col:
        flags |= nv.PT_MX_COL | (nv.PT_MX_COL_2D if col_recipe.use_2d_block else 0) | (nv.PT_MX_COL_RHT if col_recipe.use_rht else 0)
        flags |= nv.PT_MX_COL_SR if col_recipe.use_sr else 0
        q_col = torch.empty(lead + (N, M_pad // div), dtype=torch.uint8, device=x.device)
        s_col = torch.empty(lead + (N, M_pad // MX_BLOCK), dtype=torch.uint8, device=x.device)
    with nv.on_device(x.device):
        if pro is not None:
            assert G == 1 and x.dim() == 2
            _launch_fused_mx(pro, x, M, N, fmt, flags, q_row, s_row, q_col, s_col)
        else:
            nv.check(nv.lib().pt_quantize_mx(nv.ptr(x), nv.src_code(x.dtype), G, M, N, fmt, flags, nv.ptr(q_row), nv.ptr(s_row),
                                              nv.ptr(q_col), nv.ptr(s_col), nv.stream(x.device)), "quantize_mx")
    view = lambda t: None if t is None else t.view(out_dtype)
    sview = lambda t: None if t is None else t.view(torch.float8_e8m0fnu)
    q_row, s_row = _shuffled(view(q_row), sview(s_row), row_recipe if want_row else None)
    q_col, s_col = _shuffled(view(q_col), sview(s_col), col_recipe if want_col else None)
    return q_row, s_row, q_col, s_col


def _quantize_mx_impl(x, out_dtype, axis, block_size, with_trans, scaling_recipe, scaling_recipe_for_trans):
    assert block_size == MX_BLOCK, f"The block size must be {MX_BLOCK} for MX quantization"
    scaling_recipe = ScalingRecipe() if scaling_recipe is None else scaling_recipe
    if with_trans:
        assert axis is None, "The axis must be None when with_trans is True."
        scaling_recipe_for_trans = ScalingRecipe() if scaling_recipe_for_trans is None else scaling_recipe_for_trans
        return _mx_quant(x, out_dtype, True, True, scaling_recipe, scaling_recipe_for_trans)
    if x.ndim == 2:
        assert axis in (0, 1), "The axis must be 0 or 1 when with_trans is False and x is 2D."
        rowwise = axis == 1
    elif x.ndim == 3:
        assert axis in (1, 2), "The axis must be 1 or 2 when with_trans is False and x is 3D."
        rowwise = axis == 2
    else:
        raise ValueError(f"The input tensor must be 2D or 3D but got {x.ndim}D.")
    q_row, s_row, q_col, s_col = _mx_quant(x, out_dtype, rowwise, not rowwise, scaling_recipe, scaling_recipe)
    return (q_row, s_row) if rowwise else (q_col, s_col)


def quantize_mxfp8_impl(x, out_dtype, axis, block_size, with_trans=False, scaling_recipe=None,
                        scaling_recipe_for_trans=None):
    return _quantize_mx_impl(x, out_dtype, axis, block_size, with_trans, scaling_recipe, scaling_recipe_for_trans)


def quantize_mxfp4_impl(x, out_dtype, axis, block_size, with_trans=False, scaling_recipe=None,
                        scaling_recipe_for_trans=None):
    return _quantize_mx_impl(x, out_dtype, axis, block_size, with_trans, scaling_recipe, scaling_recipe_for_trans)


def _dequantize_mx(x, out_dtype, axis, scale_inv, orig_shape=None):
    """x: row-wise [R, C_pad(/2)] data (axis = last) or col-wise transposed data (axis = first, 2-D).
    Returns the dequantized tensor in the ORIGINAL orientation (col-wise inputs are re-transposed)."""
    nv.require_cuda(x, scale_inv)
    fmt = nv.fmt_code(x.dtype)
    xb = x.contiguous().view(torch.uint8)
    sb = scale_inv.contiguous().view(torch.uint8)
    lead = xb.shape[:-2]
    rows, stored = xb.shape[-2], xb.shape[-1] * (2 if fmt == nv.PT_E2M1 else 1)
    transpose = axis in (0, -2) if x.dim() == 2 else axis in (1, -2)
    cols = stored
    if orig_shape is not None:
        cols = orig_shape[-2] if transpose else orig_shape[-1]
    outs = []
    xs = xb.reshape(-1, rows, xb.shape[-1])
    ss = sb.reshape(-1, rows, sb.shape[-1])
    for g in range(xs.shape[0]):
        y = torch.empty((cols, rows) if transpose else (rows, cols), dtype=out_dtype, device=x.device)
        with nv.on_device(x.device):
            nv.check(nv.lib().pt_dequantize_mx(nv.ptr(xs[g]), fmt, nv.ptr(ss[g]), rows, cols, stored, int(transpose),
                                                nv.ptr(y), nv.src_code(out_dtype), nv.stream(x.device)), "dequantize_mx")
        outs.append(y)
    return outs[0] if not lead else torch.stack(outs).reshape(*lead, *outs[0].shape)


def dequantize_mxfp8_impl(x, out_dtype, axis, block_size, scale_inv, scaling_recipe=None, orig_shape=None):
    assert block_size == MX_BLOCK
    return _dequantize_mx(x, out_dtype, axis, scale_inv, orig_shape)


def dequantize_mxfp4_impl(x, out_dtype, axis, block_size, scale_inv, scaling_recipe=None, orig_shape=None):
    assert block_size == MX_BLOCK
    return _dequantize_mx(x, out_dtype, axis, scale_inv, orig_shape)


def transpose_2d(x: torch.Tensor) -> torch.Tensor:
    nv.require_cuda(x)
    assert x.dim() == 2
    x = x.contiguous()
    y = torch.empty((x.shape[1], x.shape[0]), dtype=x.dtype, device=x.device)
    with nv.on_device(x.device):
        nv.check(nv.lib().pt_transpose_2d(nv.ptr(x), x.shape[0], x.shape[1], x.element_size(), nv.ptr(y),
                                           nv.stream(x.device)), "transpose_2d")
    return y


def transpose_batched(x: torch.Tensor) -> torch.Tensor:
    """[B, M, N] -> [B, N, M] (contiguous), one launch for the whole batch."""
    nv.require_cuda(x)
    assert x.dim() == 3
    x = x.contiguous()
    B, M, N = x.shape
    y = torch.empty((B, N, M), dtype=x.dtype, device=x.device)
    with nv.on_device(x.device):
        nv.check(nv.lib().pt_transpose_batched(nv.ptr(x), B, M, N, x.element_size(), nv.ptr(y), nv.stream(x.device)),
                 "transpose_batched")
    return y


def grouped_transpose_pad(x: torch.Tensor, group_offs: torch.Tensor, padded_offs: torch.Tensor) -> torch.Tensor:
    """x [M, C] of 1- or 2-byte elements, grouped along M -> [C, T] with each group's tokens in its 128-padded segment
    (zero filled), T = round_up(M, 128) + 128 * G: an upper bound of padded_offs[-1] known without reading the device."""
    nv.require_cuda(x, group_offs, padded_offs)
    assert x.dim() == 2 and x.element_size() in (1, 2)
    x = x.contiguous()
    M, C = x.shape
    G = group_offs.numel() - 1
    T = ceil_div(M, BLOCK) * BLOCK + BLOCK * G
    y = torch.empty((C, T), dtype=x.dtype, device=x.device)
    with nv.on_device(x.device):
        nv.check(nv.lib().pt_grouped_transpose_pad(nv.ptr(x), M, C, x.element_size(), nv.ptr(group_offs.to(torch.int64).contiguous()),
                                                    nv.ptr(padded_offs.to(torch.int64).contiguous()), G, nv.ptr(y), T,
                                                    nv.stream(x.device)), "grouped_transpose_pad")
    return y


# ------------------------------------------------------------------------------ grouped MX
MX_GROUP_ROW_ALIGN = 32   # fp8 row-wise copy: each group padded to 32 rows (quantization.cpp:1098 of the reference)
MX_GROUP_COL_ALIGN = 128  # col-wise copy: each group padded to 128 rows


def _grouped_mx_quant(x, out_dtype, group_lens, group_offs, want_row, want_col, row_recipe, col_recipe, pro=None):
    nv.require_cuda(x, group_lens, group_offs)
    for r in (row_recipe, col_recipe):
        if r is not None and (r.shuffle_scale or r.shuffle_out):
            raise NotImplementedError("pre-shuffled MX layouts are provided for the dense quantizers only")
        if r is not None and r.use_2d_block:
            raise NotImplementedError("2-D block scales are a weight option; grouped activations use 1-D blocks")
    assert x.dim() == 2, "Input must be 2D"
    x = x.contiguous()
    fmt = nv.fmt_code(out_dtype)
    fp4 = fmt == nv.PT_E2M1
    for r in (row_recipe, col_recipe):
        if r is not None and r.use_sr and not fp4:
            raise ValueError("stochastic rounding is an MXFP4 option (ScalingRecipe.use_sr)")
    M, N = x.shape
    if pro is not None:
        N //= 2
    G = group_lens.numel()
    lens = group_lens.to(torch.int64).contiguous()
    offs = group_offs.to(torch.int64).contiguous()
    N_pad = ceil_div(N, MX_ALIGN) * MX_ALIGN
    div = 2 if fp4 else 1
    row_align = 1 if fp4 else MX_GROUP_ROW_ALIGN
    if fp4:
        plens_row, poffs_row = lens, offs
        rows_alloc = M
    else:
        plens_row, poffs_row = compute_padded_group_offs(lens, row_align)
        rows_alloc = ceil_div(M + G * row_align, row_align) * row_align
    # fp4: a GEMM stage spans 256 elements of the contraction, so token segments are padded to 256
    col_align = 2 * MX_GROUP_COL_ALIGN if fp4 else MX_GROUP_COL_ALIGN
    plens_col, poffs_col = compute_padded_group_offs(lens, col_align)
    col_alloc = ceil_div(M + G * col_align, col_align) * col_align
    flags = 0
    q_row = s_row = q_col = s_col = None
    if want_row:
        flags |= nv.PT_MX_ROW | (nv.PT_MX_ROW_RHT if row_recipe.use_rht else 0) | (nv.PT_MX_ROW_SR if row_recipe.use_sr else 0)
        q_row = torch.empty((rows_alloc, N_pad // div), dtype=torch.uint8, device=x.device)
        s_row = torch.empty((rows_alloc, N_pad // MX_BLOCK), dtype=torch.uint8, device=x.device)
    if want_col:
        flags |= nv.PT_MX_COL | (nv.PT_MX_COL_RHT if col_recipe.use_rht else 0) | (nv.PT_MX_COL_SR if col_recipe.use_sr else 0)
        q_col = torch.empty((N, col_alloc // div), dtype=torch.uint8, device=x.device)
        s_col = torch.empty((N, col_alloc // MX_BLOCK), dtype=torch.uint8, device=x.device)
    with nv.on_device(x.device):
        if pro is not None:
            _launch_fused_mx(pro, x, M, N, fmt, flags, q_row, s_row, q_col, s_col, grouped=(G, offs, poffs_row, poffs_col, col_alloc))
        else:
            nv.check(nv.lib().pt_grouped_quantize_mx(nv.ptr(x), nv.src_code(x.dtype), M, N, G, nv.ptr(offs), nv.ptr(poffs_row),
                                                      nv.ptr(poffs_col), fmt, flags, nv.ptr(q_row), nv.ptr(s_row), nv.ptr(q_col),
                                                      nv.ptr(s_col), col_alloc, nv.stream(x.device)), "grouped_quantize_mx")
    view = lambda t: None if t is None else t.view(out_dtype)
    sview = lambda t: None if t is None else t.view(torch.float8_e8m0fnu)
    return (view(q_row), sview(s_row), view(q_col), sview(s_col), plens_row, poffs_row, plens_col, poffs_col)


def _grouped_quantize_mx_impl(x, out_dtype, axis, block_size, group_lens, group_offs, with_trans, scaling_recipe,
                              scaling_recipe_for_trans):
    assert block_size == MX_BLOCK, f"The block size must be {MX_BLOCK} for MX quantization"
    scaling_recipe = ScalingRecipe() if scaling_recipe is None else scaling_recipe
    if with_trans:
        scaling_recipe_for_trans = ScalingRecipe() if scaling_recipe_for_trans is None else scaling_recipe_for_trans
        return _grouped_mx_quant(x, out_dtype, group_lens, group_offs, True, True, scaling_recipe, scaling_recipe_for_trans)
    assert axis in (0, 1), "The axis must be 0 or 1 when with_trans is False."
    q_row, s_row, q_col, s_col, lr, orow, lc, ocol = _grouped_mx_quant(x, out_dtype, group_lens, group_offs, axis == 1,
                                                                       axis == 0, scaling_recipe, scaling_recipe)
    return (q_row, s_row, lr, orow) if axis == 1 else (q_col, s_col, lc, ocol)


def grouped_quantize_mxfp8_impl(x, out_dtype, axis, block_size, group_lens, group_offs, with_trans=False,
                                scaling_recipe=None, scaling_recipe_for_trans=None):
    """(q, s, lens_padded, offs_padded), or with_trans: (q_row, s_row, q_col, s_col, lens_pad_row, offs_pad_row,
    lens_pad_col, offs_pad_col).  Row copy: groups padded to 32 rows; col copy (transposed): groups padded to 128."""
    return _grouped_quantize_mx_impl(x, out_dtype, axis, block_size, group_lens, group_offs, with_trans, scaling_recipe,
                                     scaling_recipe_for_trans)


def grouped_quantize_mxfp4_impl(x, out_dtype, axis, block_size, group_lens, group_offs, with_trans=False,
                                scaling_recipe=None, scaling_recipe_for_trans=None):
    """As the fp8 form with packed e2m1; the row copy is tight (row i = input row i)."""
    return _grouped_quantize_mx_impl(x, out_dtype, axis, block_size, group_lens, group_offs, with_trans, scaling_recipe,
                                     scaling_recipe_for_trans)


def _tight_row_index(group_offs, group_offs_padded, total_M, device):
    """For every row r of the tight (un-padded) layout, the row of the padded layout that holds it; built on the
    device from the two offset arrays."""
    offs = group_offs.to(torch.int64)
    r = torch.arange(total_M, dtype=torch.int64, device=device)
    g = torch.searchsorted(offs[1:].contiguous(), r, right=True).clamp_(max=offs.numel() - 2)
    return group_offs_padded.to(torch.int64)[g] + (r - offs[g])


def grouped_dequantize_mxfp8_impl(x: torch.Tensor, out_dtype: torch.dtype, axis: int, block_size: int, scale_inv: torch.Tensor,
                                  group_offs: torch.Tensor, group_offs_padded: torch.Tensor,
                                  total_M: Optional[int] = None) -> torch.Tensor:
    """Undoes grouped_quantize_mxfp8_impl: x is the row-wise copy [M_pad, N] (axis 1) or the column-wise, transposed copy
    [N, M_pad] (axis 0), both with per-group padded token segments at `group_offs_padded`; returns the tight
    [total_M, N] tensor.  Same call shape as the reference (kernels/quantization/quantization_impl.py:838-865); like
    there, total_M = None costs a host read of group_offs[-1]."""
    nv.require_cuda(x, scale_inv, group_offs, group_offs_padded)
    assert block_size == MX_BLOCK
    assert x.dim() == 2 and scale_inv.dim() == 2 and axis in (0, 1)
    assert out_dtype in (torch.float16, torch.bfloat16, torch.float32)
    if total_M is None:
        total_M = int(group_offs[-1].item())
    padded = _dequantize_mx(x, out_dtype, axis, scale_inv)      # [M_pad, N(_pad)] in the original orientation
    idx = _tight_row_index(group_offs, group_offs_padded, total_M, x.device)
    return padded.index_select(0, idx)


# ------------------------------------------------------------------------------ operator + MX quantizer in one pass
def _glu_recipes(out_dtype, col_rht):
    if col_rht:
        assert nv.fmt_code(out_dtype) == nv.PT_E2M1, "the Hadamard transform of the transposed copy is an MXFP4 option"
    return ScalingRecipe(), ScalingRecipe(use_rht=bool(col_rht))


def glu_quantize_mx_impl(x: torch.Tensor, probs: torch.Tensor, row_mask, act: str, out_dtype, fused=None, col_rht=False):
    """MX copies (row-wise and transposed) of act(x[:, :H]) * x[:, H:] * probs without the [tokens, H] intermediate:
    (q_row, s_row, q_col, s_col), the bytes `glu_fwd_with_probs` followed by `quantize_mx*_impl(with_trans=True)` gives.
    fused=None picks the one-pass kernel where it applies; False forces the two kernels (the comparison the tests make)."""
    from ..activation.glu_impl import ACT_CODES, glu_fwd_with_probs
    nv.require_cuda(x, probs, row_mask)
    x, probs = x.contiguous(), probs.contiguous().view(-1)
    H = x.shape[1] // 2
    use = fused_mx_supported(x, H, out_dtype, True) if fused is None else fused
    row_r, col_r = _glu_recipes(out_dtype, col_rht)
    if not use:
        return _mx_quant(glu_fwd_with_probs(x, probs, row_mask, act), out_dtype, True, True, row_r, col_r)
    return _mx_quant(x, out_dtype, True, True, row_r, col_r, pro=("glu", probs, row_mask, ACT_CODES[act]))


def grouped_glu_quantize_mx_impl(x, probs, row_mask, act: str, out_dtype, group_lens, group_offs, fused=None, col_rht=False):
    """Grouped form (token segments per expert); returns what `grouped_quantize_mx*_impl(with_trans=True)` returns."""
    from ..activation.glu_impl import ACT_CODES, glu_fwd_with_probs
    nv.require_cuda(x, probs, row_mask)
    x, probs = x.contiguous(), probs.contiguous().view(-1)
    H = x.shape[1] // 2
    use = (fused_mx_supported(x, H, out_dtype, True) and group_lens.numel() <= 256) if fused is None else fused
    row_r, col_r = _glu_recipes(out_dtype, col_rht)
    if not use:
        return _grouped_mx_quant(glu_fwd_with_probs(x, probs, row_mask, act), out_dtype, group_lens, group_offs, True, True, row_r, col_r)
    return _grouped_mx_quant(x, out_dtype, group_lens, group_offs, True, True, row_r, col_r, pro=("glu", probs, row_mask, ACT_CODES[act]))


def glu_quantize_mx_row_impl(x: torch.Tensor, probs: torch.Tensor, row_mask, act: str, out_dtype, fused=None):
    """Row-wise MX copy of act(x[:, :H]) * x[:, H:] * probs, (q_row, s_row), in one pass over x: what a forward-only caller
    feeds the down projection.  Falls back to activation kernel + row-wise quantizer outside the one-pass kernel's range
    (bf16, H a multiple of 32); both write the same bytes."""
    from ..activation.glu_impl import ACT_CODES, glu_fwd_with_probs
    nv.require_cuda(x, probs, row_mask)
    x = x.reshape(-1, x.shape[-1])
    rows, h2 = x.shape
    assert h2 % 2 == 0
    H = h2 // 2
    ok = x.dtype == torch.bfloat16 and H % MX_BLOCK == 0
    use = ok if fused is None else fused
    if use:
        x, probs = x.contiguous(), probs.contiguous().view(-1)
        fmt = nv.fmt_code(out_dtype)
        n_pad = ceil_div(H, MX_ALIGN) * MX_ALIGN
        q = torch.empty(rows, n_pad // (2 if fmt == nv.PT_E2M1 else 1), dtype=torch.uint8, device=x.device)
        s = torch.empty(rows, n_pad // MX_BLOCK, dtype=torch.uint8, device=x.device)
        with nv.on_device(x.device):
            nv.check(nv.lib().pt_glu_quantize_mx_row(nv.ptr(x), nv.src_code(x.dtype), nv.ptr(probs), nv.ptr(row_mask), rows, H, ACT_CODES[act], fmt,
                                                      nv.ptr(q), nv.ptr(s), nv.stream(x.device)), "glu_quantize_mx_row")
        return q.view(out_dtype), s.view(torch.float8_e8m0fnu)
    q, s, _, _ = _mx_quant(glu_fwd_with_probs(x, probs, row_mask, act), out_dtype, True, False, ScalingRecipe(), ScalingRecipe())
    return q, s


def rmsnorm_quantize_mx_row_impl(x: torch.Tensor, gamma: torch.Tensor, eps: float, zero_centered: bool, out_dtype, fused=None):
    """Row-wise MX copy of rmsnorm(x) and the row statistics, (q_row, s_row, rstd), in one pass over x: what a forward-only
    caller feeds the first GEMM.  Falls back to RMSNorm kernel + row-wise quantizer outside the one-pass kernel's range
    (bf16, H a multiple of 32, at most 8192); both write the same bytes."""
    from ..normalization.rmsnorm_impl import rmsnorm_fwd_impl
    nv.require_cuda(x, gamma)
    x2 = x.reshape(-1, x.shape[-1]).contiguous()
    gamma = gamma.contiguous()
    rows, H = x2.shape
    ok = x2.dtype == torch.bfloat16 and gamma.dtype == torch.bfloat16 and H % MX_BLOCK == 0 and H <= 8192
    use = ok if fused is None else fused
    if use:
        fmt = nv.fmt_code(out_dtype)
        n_pad = ceil_div(H, MX_ALIGN) * MX_ALIGN
        q = torch.empty(rows, n_pad // (2 if fmt == nv.PT_E2M1 else 1), dtype=torch.uint8, device=x.device)
        s = torch.empty(rows, n_pad // MX_BLOCK, dtype=torch.uint8, device=x.device)
        rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
        with nv.on_device(x.device):
            nv.check(nv.lib().pt_rmsnorm_quantize_mx_row(nv.ptr(x2), nv.src_code(x2.dtype), nv.ptr(gamma), float(eps), int(bool(zero_centered)),
                                                          rows, H, fmt, nv.ptr(q), nv.ptr(s), nv.ptr(rstd), nv.stream(x.device)),
                     "rmsnorm_quantize_mx_row")
        return q.view(out_dtype), s.view(torch.float8_e8m0fnu), rstd
    y, _, rstd = rmsnorm_fwd_impl(x2, gamma, eps, zero_centered)
    q, s, _, _ = _mx_quant(y, out_dtype, True, False, ScalingRecipe(), ScalingRecipe())
    return q, s, rstd


def rmsnorm_quantize_mx_impl(x: torch.Tensor, gamma: torch.Tensor, eps: float, zero_centered: bool, out_dtype, fused=None):
    """MX copies of rmsnorm(x) and the row statistics: (q_row, s_row, q_col, s_col, rstd).  One statistics pass over x,
    then the quantizer normalises each tile as it loads it; the normalised tensor is never written."""
    from ..normalization.rmsnorm_impl import rmsnorm_fwd_impl, rmsnorm_stats_impl
    nv.require_cuda(x, gamma)
    x2 = x.reshape(-1, x.shape[-1]).contiguous()
    gamma = gamma.contiguous()
    use = (fused_mx_supported(x2, x2.shape[1], out_dtype, False) and gamma.dtype == x2.dtype) if fused is None else fused
    if not use:
        y, _, rstd = rmsnorm_fwd_impl(x2, gamma, eps, zero_centered)
        return (*_mx_quant(y, out_dtype, True, True, ScalingRecipe(), ScalingRecipe()), rstd)
    rstd = rmsnorm_stats_impl(x2, eps)
    return (*_mx_quant(x2, out_dtype, True, True, ScalingRecipe(), ScalingRecipe(), pro=("rmsnorm", rstd, gamma, zero_centered)), rstd)
