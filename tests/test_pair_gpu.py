"""The CTA-pair GEMM kernels (two CTAs per 256-row tile) against the single-CTA kernels on the same quantized operands:
dense, grouped (uneven groups with a short and an empty one) and variable-K forms, FP8 tensorwise / MXFP8 / MXFP4.
Both kernels sum K in the same order, so the outputs must agree to fp32 rounding of the accumulator (checked as a
relative Frobenius distance <= 1e-6); the single-CTA kernels are checked against the oracle elsewhere.  The
environment variable PT_GEMM_PAIR=0 selects the single-CTA kernel for a call."""
import os

import pytest
import torch

from oracle import gemm as og
from tests._util import f32, make

pytestmark = pytest.mark.gpu

F8 = torch.float8_e4m3fn
F4 = torch.float4_e2m1fn_x2
LENS = [3000, 100, 0, 2500, 4096, 1024, 3616, 2048]   # 16384 rows, average 2048 per group


@pytest.fixture(scope="module")
def m():
    from primus_turbo.pytorch.core.low_precision import ScalingGranularity, ScalingRecipe
    from primus_turbo.pytorch.kernels import _native as nv
    from primus_turbo.pytorch.kernels.gemm import gemm_fp8_impl as gi
    from primus_turbo.pytorch.kernels.grouped_gemm import grouped_gemm_fp4_impl as gg4
    from primus_turbo.pytorch.kernels.grouped_gemm import grouped_gemm_fp8_impl as ggi
    from primus_turbo.pytorch.kernels.quantization import quantization_impl as qi
    return dict(qi=qi, gi=gi, ggi=ggi, gg4=gg4, nv=nv, SG=ScalingGranularity, SR=ScalingRecipe)


def _both(fn):
    """fn() with the pair kernels and with the single-CTA kernels (the block-scaled pair kernel is opt-in)."""
    old = {k: os.environ.get(k) for k in ("PT_GEMM_PAIR", "PT_BW_GEMM_PAIR")}
    try:
        os.environ["PT_GEMM_PAIR"] = "1"
        os.environ["PT_BW_GEMM_PAIR"] = "1"
        pair = fn()
        os.environ["PT_GEMM_PAIR"] = "0"
        single = fn()
    finally:
        for k, v in old.items():
            if v is None:
                os.environ.pop(k, None)
            else:
                os.environ[k] = v
    torch.cuda.synchronize()
    return pair, single


def _offs(lens):
    lens_t = torch.tensor(lens, dtype=torch.int64, device="cuda")
    offs = torch.zeros(len(lens) + 1, dtype=torch.int64, device="cuda")
    offs[1:] = torch.cumsum(lens_t, 0)
    return lens_t, offs


def _close(a, b):
    assert a.shape == b.shape
    assert og.rel_frobenius(f32(a), f32(b)) <= 1e-6


@pytest.mark.parametrize("M,N,K", [(4096, 4096, 1024), (4000, 4360, 640), (1024, 16384, 512), (4100, 4104, 1104)])
@pytest.mark.parametrize("gran", ["tensorwise", "rowwise", "mx"])
def test_dense_pair_matches_single(m, M, N, K, gran):
    qi, gi, nv, SG = m["qi"], m["gi"], m["nv"], m["SG"]
    if gran == "mx" and K % 128:
        pytest.skip("MX operands are padded to 128 along K by their quantizer; covered by the other shapes")
    a, w = make((M, K), torch.bfloat16, 71, "outlier"), make((N, K), torch.bfloat16, 72, "weight")
    if gran == "tensorwise":
        (qa, sa), (qw, sw), g = qi.quantize_fp8_tensorwise_impl(a, F8), qi.quantize_fp8_tensorwise_impl(w, F8), SG.TENSORWISE
    elif gran == "rowwise":
        (qa, sa), (qw, sw), g = qi.quantize_fp8_rowwise_impl(a, F8, -1), qi.quantize_fp8_rowwise_impl(w, F8, -1), SG.ROWWISE
    else:
        (qa, sa), (qw, sw), g = qi.quantize_mxfp8_impl(a, F8, 1, 32), qi.quantize_mxfp8_impl(w, F8, 1, 32), SG.MX_BLOCKWISE
    pair, single = _both(lambda: gi.gemm_fp8_impl(qa, sa, False, qw, sw, True, torch.float32, False, g))
    nv.check_status(pair.device)
    _close(pair, single)


def test_grouped_mxfp8_pair_matches_single(m):
    qi, ggi, nv, SG, SR = m["qi"], m["ggi"], m["nv"], m["SG"], m["SR"]
    lens_t, offs = _offs(LENS)
    G, M, K, N = len(LENS), sum(LENS), 1024, 2240
    a = make((M, K), torch.bfloat16, 73, "outlier")
    w = make((G, N, K), torch.bfloat16, 74, "weight")
    a_row, a_s_row, a_col, a_s_col, _, orow, lcol, ocol = qi.grouped_quantize_mxfp8_impl(a, F8, None, 32, lens_t, offs, with_trans=True)
    two_d = SR(use_2d_block=True)
    w_row, w_s_row = qi.quantize_mxfp8_impl(w, F8, 2, 32, scaling_recipe=two_d)
    pair, single = _both(lambda: ggi.grouped_gemm_fp8_impl(a_row, w_row, a_s_row, w_s_row, lens_t, orow, False, True, torch.float32,
                                                           SG.MX_BLOCKWISE, group_offs_out=offs))
    nv.check_status(pair.device)
    _close(pair, single)
    # variable-K (grouped wgrad): every group contracts its own token range
    go = make((M, N), torch.bfloat16, 75, "small")
    _, _, g_col, g_s_col, _, _, lcol, ocol = qi.grouped_quantize_mxfp8_impl(go, torch.float8_e5m2, None, 32, lens_t, offs, with_trans=True)
    pair, single = _both(lambda: ggi.grouped_gemm_fp8_variable_k_impl(g_col, a_col, g_s_col, a_s_col, lcol, ocol, False, False, False,
                                                                      torch.float32, SG.MX_BLOCKWISE))
    nv.check_status(pair.device)
    _close(pair, single)


def test_grouped_tensorwise_pair_matches_single(m):
    qi, ggi, nv, SG = m["qi"], m["ggi"], m["nv"], m["SG"]
    lens_t, offs = _offs(LENS)
    G, M, K, N = len(LENS), sum(LENS), 1024, 2048
    a = make((M, K), torch.bfloat16, 76, "outlier")
    w = make((G, N, K), torch.bfloat16, 77, "weight")
    (qa, sa), (qw, sw) = qi.quantize_fp8_tensorwise_impl(a, F8), qi.quantize_fp8_tensorwise_impl(w, F8)
    pair, single = _both(lambda: ggi.grouped_gemm_fp8_impl(qa, qw, sa, sw, lens_t, offs, False, True, torch.bfloat16, SG.TENSORWISE))
    nv.check_status(pair.device)
    assert torch.equal(pair, single)


def test_grouped_mxfp4_pair_matches_single(m):
    qi, gg4, nv, SR = m["qi"], m["gg4"], m["nv"], m["SR"]
    lens_t, offs = _offs(LENS)
    G, M, K, N = len(LENS), sum(LENS), 1024, 2240
    a = make((M, K), torch.bfloat16, 78, "outlier")
    w = make((G, N, K), torch.bfloat16, 79, "weight")
    a_row, a_s_row, a_col, a_s_col, _, orow, lcol, ocol = qi.grouped_quantize_mxfp4_impl(a, F4, None, 32, lens_t, offs, with_trans=True)
    w_row, w_s_row = qi.quantize_mxfp4_impl(w, F4, 2, 32, scaling_recipe=SR(use_2d_block=True))
    pair, single = _both(lambda: gg4.grouped_gemm_fp4_impl(a_row, w_row, a_s_row, w_s_row, lens_t, orow, out_dtype=torch.float32,
                                                           group_offs_out=offs))
    nv.check_status(pair.device)
    _close(pair, single)
    go = make((M, N), torch.bfloat16, 80)
    _, _, g_col, g_s_col, _, _, lcol, ocol = qi.grouped_quantize_mxfp4_impl(go, F4, None, 32, lens_t, offs, with_trans=True)
    pair, single = _both(lambda: gg4.grouped_gemm_fp4_variable_k_impl(g_col, a_col, g_s_col, a_s_col, lcol, ocol, torch.float32))
    nv.check_status(pair.device)
    _close(pair, single)


@pytest.mark.parametrize("M,N,K", [(4096, 4096, 1024), (4000, 4360, 640), (1024, 16384, 512)])
def test_dense_blockwise_pair_matches_single(m, M, N, K):
    """Block-scaled GEMM on CTA pairs: forward (K-major operands, 128 x 128 weight scales), dgrad (the weight read in
    place as an MN-major operand) and wgrad (both operands MN-major, per-column scales) against the single-CTA kernel."""
    qi, gi, SG = m["qi"], m["gi"], m["SG"]
    a = make((M, K), torch.bfloat16, 61, "normal")
    w = make((N, K), torch.bfloat16, 62, "normal")
    g = make((M, N), torch.bfloat16, 63, "normal")
    a_row, a_s_row, a_col, a_s_col = qi.quant_fp8_blockwise_dual_impl(a, F8, 128)
    g_row, g_s_row, g_col, g_s_col = qi.quant_fp8_blockwise_dual_impl(g, F8, 128)
    w_q, w_s = qi.quant_fp8_blockwise_for_weight_impl(w, F8)
    fwd = _both(lambda: gi.gemm_fp8_impl(a_row, a_s_row, False, w_q, w_s, True, torch.bfloat16, False, SG.BLOCKWISE))
    _close(*fwd)
    dgrad = _both(lambda: gi.gemm_fp8_impl(g_row, g_s_row, False, w_q, w_s, False, torch.bfloat16, False, SG.BLOCKWISE))
    _close(*dgrad)
    wgrad = _both(lambda: gi.gemm_fp8_impl(g_col, g_s_col, True, a_col, a_s_col, False, torch.float32, False, SG.BLOCKWISE))
    _close(*wgrad)


def test_grouped_blockwise_pair_matches_single(m):
    qi, ggi, SG = m["qi"], m["ggi"], m["SG"]
    lens_t, offs = _offs(LENS)
    M, K, N, G = sum(LENS), 512, 1024, len(LENS)
    a = make((M, K), torch.bfloat16, 64, "normal")
    w = make((G, N, K), torch.bfloat16, 65, "normal")
    g = make((M, N), torch.bfloat16, 66, "normal")
    a_row, a_col, a_s_row, a_s_col, vk_lens, vk_offs = qi.quant_fp8_blockwise_segment_m_row_col_impl(a, F8, 128, lens_t, offs)
    g_row, g_col, g_s_row, g_s_col, _, _ = qi.quant_fp8_blockwise_segment_m_row_col_impl(g, F8, 128, lens_t, offs)
    w_q, w_s = qi.quant_fp8_blockwise_for_weight_impl(w, F8)
    fwd = _both(lambda: ggi.grouped_gemm_fp8_impl(a_row, w_q, a_s_row, w_s, lens_t, offs, False, True, torch.bfloat16, SG.BLOCKWISE))
    _close(*fwd)
    dgrad = _both(lambda: ggi.grouped_gemm_fp8_impl(g_row, w_q, g_s_row, w_s, lens_t, offs, False, False, torch.bfloat16, SG.BLOCKWISE))
    _close(*dgrad)
    wgrad = _both(lambda: ggi.grouped_gemm_fp8_variable_k_impl(a_col, g_col, a_s_col, g_s_col, vk_lens, vk_offs, True, False, True,
                                                               torch.bfloat16, SG.BLOCKWISE))
    _close(*wgrad)
