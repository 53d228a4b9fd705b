"""Dense FP8 / MXFP8 GEMM through the C ABI against the fp32-dequantized matmul of the oracle.
Tolerance (stated by the task): relative Frobenius error <= 1e-2 for FP8; the reference's own SNR
gates against the unquantized product (tests/pytorch/ops/test_gemm_fp8.py:101-114) are checked too."""
import numpy as np
import pytest
import torch

from oracle import gemm as og
from oracle import quant as oq
from tests._util import f32, fmt_of, make, u8

pytestmark = pytest.mark.gpu

FP8_TOL = 1e-2


@pytest.fixture(scope="module")
def mods():
    from primus_turbo.pytorch.core.low_precision import ScalingGranularity, ScalingRecipe
    from primus_turbo.pytorch.kernels import _native as nv
    from primus_turbo.pytorch.kernels.gemm import gemm_fp8_impl as gi
    from primus_turbo.pytorch.kernels.quantization import quantization_impl as qi
    return qi, gi, nv, ScalingGranularity, ScalingRecipe


def _ref(qa, sa, qb, sb, fa, fb):
    return og.gemm_nt(oq.dequantize_fp8(qa, sa, fa), oq.dequantize_fp8(qb, sb, fb))


@pytest.mark.parametrize("M,N,K", [(128, 128, 128), (256, 512, 256), (255, 520, 576), (507, 1024, 2048), (1000, 264, 144)])
@pytest.mark.parametrize("fa,fb", [(torch.float8_e4m3fn, torch.float8_e4m3fn), (torch.float8_e5m2, torch.float8_e4m3fn)])
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
def test_tensorwise_nt(mods, M, N, K, fa, fb, out_dtype):
    qi, gi, nv, SG, _ = mods
    a, b = make((M, K), torch.bfloat16, 21), make((N, K), torch.bfloat16, 22)
    qa, sa = qi.quantize_fp8_tensorwise_impl(a, fa)
    qb, sb = qi.quantize_fp8_tensorwise_impl(b, fb)
    c = gi.gemm_fp8_impl(qa, sa, False, qb, sb, True, out_dtype, False, SG.TENSORWISE)
    nv.check_status(c.device)
    ref = _ref(u8(qa), f32(sa), u8(qb), f32(sb), fmt_of(fa), fmt_of(fb))
    err = og.rel_frobenius(f32(c), ref)
    assert err <= (FP8_TOL if out_dtype == torch.bfloat16 else 1e-5), err
    if fa == torch.float8_e4m3fn:
        assert og.snr_db(f32(c), f32(a) @ f32(b).T) > 25


@pytest.mark.parametrize("block_n", [128, 240, 256])
def test_tile_widths_agree(mods, block_n):
    qi, gi, nv, SG, _ = mods
    a, b = make((384, 512), torch.bfloat16, 23), make((1000, 512), torch.bfloat16, 24)
    qa, sa = qi.quantize_fp8_tensorwise_impl(a, torch.float8_e4m3fn)
    qb, sb = qi.quantize_fp8_tensorwise_impl(b, torch.float8_e4m3fn)
    c = gi.gemm_fp8_impl(qa, sa, False, qb, sb, True, torch.float32, False, SG.TENSORWISE, block_n=block_n)
    nv.check_status(c.device)
    ref = _ref(u8(qa), f32(sa), u8(qb), f32(sb), "e4m3", "e4m3")
    assert og.rel_frobenius(f32(c), ref) <= 1e-5


@pytest.mark.parametrize("trans_a,trans_b,trans_c", [(False, False, False), (True, False, False), (False, True, True),
                                                     (True, True, False), (False, False, True)])
def test_tensorwise_layouts(mods, trans_a, trans_b, trans_c):
    qi, gi, nv, SG, _ = mods
    M, N, K = 256, 384, 512
    a = make((K, M) if trans_a else (M, K), torch.bfloat16, 25)
    b = make((N, K) if trans_b else (K, N), torch.bfloat16, 26)
    qa, sa = qi.quantize_fp8_tensorwise_impl(a, torch.float8_e4m3fn)
    qb, sb = qi.quantize_fp8_tensorwise_impl(b, torch.float8_e4m3fn)
    c = gi.gemm_fp8_impl(qa, sa, trans_a, qb, sb, trans_b, torch.float32, trans_c, SG.TENSORWISE)
    nv.check_status(c.device)
    da = oq.dequantize_fp8(u8(qa), f32(sa), "e4m3")
    db = oq.dequantize_fp8(u8(qb), f32(sb), "e4m3")
    ref = (da.T if trans_a else da) @ (db.T if trans_b else db)
    ref = ref.T if trans_c else ref
    assert og.rel_frobenius(f32(c), ref) <= 1e-5


@pytest.mark.parametrize("M,N,K", [(256, 384, 512), (144, 272, 200), (1040, 528, 1000), (4096, 4096, 2048), (250, 384, 512)])
@pytest.mark.parametrize("which", ["dgrad", "wgrad"])
def test_rowwise_backward_layouts_read_in_place(mods, M, N, K, which):
    """The two backward GEMMs of a rowwise linear with their operands as the forward stored them (MN-major in place when
    the row counts are multiples of 16, the transposed-copy path for M = 250): dgrad = g [M, N] . w [N, K] contracts over
    N, wgrad = g^T . x contracts over the tokens; scales run along the non-contracted index of each operand."""
    qi, gi, nv, SG, _ = mods
    x, w, g = make((M, K), torch.bfloat16, 41, "outlier"), make((N, K), torch.bfloat16, 42, "weight"), make((M, N), torch.bfloat16, 43)
    if which == "dgrad":
        qg, sg = qi.quantize_fp8_rowwise_impl(g, torch.float8_e5m2, -1)          # per token
        qw, sw = qi.quantize_fp8_rowwise_impl(w, torch.float8_e4m3fn, -2)        # per input feature
        c = gi.gemm_fp8_impl(qg, sg, False, qw, sw, False, torch.bfloat16, False, SG.ROWWISE)      # [M, K]
        da = oq.dequantize_fp8(u8(qg), f32(sg).reshape(-1, 1), "e5m2")
        db = oq.dequantize_fp8(u8(qw), f32(sw).reshape(1, -1), "e4m3")
        ref, exact = da @ db, f32(g) @ f32(w)
    else:
        qx, sx = qi.quantize_fp8_rowwise_impl(x, torch.float8_e4m3fn, -2)        # per input feature
        qg, sg = qi.quantize_fp8_rowwise_impl(g, torch.float8_e5m2, -2)          # per output feature
        c = gi.gemm_fp8_impl(qx, sx, True, qg, sg, False, torch.bfloat16, True, SG.ROWWISE)        # [N, K]
        da = oq.dequantize_fp8(u8(qx), f32(sx).reshape(1, -1), "e4m3")
        db = oq.dequantize_fp8(u8(qg), f32(sg).reshape(1, -1), "e5m2")
        ref, exact = db.T @ da, f32(g).T @ f32(x)
    nv.check_status(c.device)
    assert og.rel_frobenius(f32(c), ref) <= FP8_TOL
    assert og.snr_db(f32(c), exact) > 20


@pytest.mark.parametrize("M,N,K", [(256, 512, 256), (255, 520, 576), (512, 4096, 1024)])
def test_rowwise_nt(mods, M, N, K):
    qi, gi, nv, SG, _ = mods
    a, b = make((M, K), torch.bfloat16, 27, "outlier"), make((N, K), torch.bfloat16, 28, "weight")
    qa, sa = qi.quantize_fp8_rowwise_impl(a, torch.float8_e4m3fn, -1)
    qb, sb = qi.quantize_fp8_rowwise_impl(b, torch.float8_e4m3fn, -1)
    c = gi.gemm_fp8_impl(qa, sa, False, qb, sb, True, torch.bfloat16, False, SG.ROWWISE)
    nv.check_status(c.device)
    ref = _ref(u8(qa), f32(sa), u8(qb), f32(sb), "e4m3", "e4m3")
    assert og.rel_frobenius(f32(c), ref) <= FP8_TOL
    assert og.snr_db(f32(c), f32(a) @ f32(b).T) > 25


@pytest.mark.parametrize("M,N,K", [(128, 128, 128), (256, 512, 256), (255, 520, 576), (507, 1000, 2048), (2048, 4096, 1024)])
@pytest.mark.parametrize("fa,fb", [(torch.float8_e4m3fn, torch.float8_e4m3fn), (torch.float8_e5m2, torch.float8_e4m3fn)])
@pytest.mark.parametrize("block_n", [0, 128, 256])
def test_mx_nt(mods, M, N, K, fa, fb, block_n):
    qi, gi, nv, SG, SR = mods
    a, b = make((M, K), torch.bfloat16, 29, "outlier"), make((N, K), torch.bfloat16, 30, "weight")
    qa, sa = qi.quantize_mxfp8_impl(a, fa, 1, 32)
    qb, sb = qi.quantize_mxfp8_impl(b, fb, 1, 32, scaling_recipe=SR(use_2d_block=True))
    c = gi.gemm_fp8_impl(qa, sa, False, qb, sb, True, torch.float32, False, SG.MX_BLOCKWISE, block_n=block_n)
    nv.check_status(c.device)
    ref = og.gemm_nt(oq.dequantize_mx(u8(qa), u8(sa), fmt_of(fa)), oq.dequantize_mx(u8(qb), u8(sb), fmt_of(fb)))
    err = og.rel_frobenius(f32(c), ref)
    assert err <= 1e-5, err   # products and power-of-two scales are exact; only fp32 summation order differs
    cb = gi.gemm_fp8_impl(qa, sa, False, qb, sb, True, torch.bfloat16, False, SG.MX_BLOCKWISE, block_n=block_n)
    assert og.rel_frobenius(f32(cb), ref) <= FP8_TOL
    if fa == torch.float8_e4m3fn:
        assert og.snr_db(f32(cb), f32(a) @ f32(b).T) > 25


def test_mx_deterministic(mods):
    # tests/pytorch/ops/test_gemm_fp8.py:190-200 of the reference: repeated runs are bit-identical
    qi, gi, nv, SG, _ = mods
    a, b = make((512, 1024), torch.bfloat16, 31), make((768, 1024), torch.bfloat16, 32)
    qa, sa = qi.quantize_mxfp8_impl(a, torch.float8_e4m3fn, 1, 32)
    qb, sb = qi.quantize_mxfp8_impl(b, torch.float8_e4m3fn, 1, 32)
    first = gi.gemm_fp8_impl(qa, sa, False, qb, sb, True, torch.bfloat16, False, SG.MX_BLOCKWISE)
    for _ in range(9):
        again = gi.gemm_fp8_impl(qa, sa, False, qb, sb, True, torch.bfloat16, False, SG.MX_BLOCKWISE)
        assert torch.equal(first, again)
    nv.check_status(first.device)


def test_large_gemms_repeat_bit_identically(mods):
    """Sizes that keep every SM busy for many tiles (CTA pairs for MX, the promotion warps of the blockwise kernel in all
    three directions): ten launches each must agree bit for bit, so that a hand-over between warp roles that is lost now
    and then does not hide behind a tolerance."""
    qi, gi, nv, SG, _ = mods
    f8, f5 = torch.float8_e4m3fn, torch.float8_e5m2
    M, N, K = 4096, 3584, 2048
    x, w, dy = make((M, K), torch.bfloat16, 41), make((N, K), torch.bfloat16, 42), make((M, N), torch.bfloat16, 43)
    qa, sa = qi.quantize_mxfp8_impl(x, f8, 1, 32)
    qb, sb = qi.quantize_mxfp8_impl(w, f8, 1, 32)
    a_row, a_row_s, a_col, a_col_s = qi.quant_fp8_blockwise_dual_impl(x, f8)
    w_q, w_s = qi.quant_fp8_blockwise_for_weight_impl(w, f8)
    g_row, g_row_s, g_col, g_col_s = qi.quant_fp8_blockwise_dual_impl(dy, f5)
    runs = [
        lambda: gi.gemm_fp8_impl(qa, sa, False, qb, sb, True, torch.bfloat16, False, SG.MX_BLOCKWISE),
        lambda: gi.gemm_fp8_impl(a_row, a_row_s, False, w_q, w_s, True, torch.bfloat16, False, SG.BLOCKWISE),
        lambda: gi.gemm_fp8_impl(g_row, g_row_s, False, w_q, w_s, False, torch.bfloat16, False, SG.BLOCKWISE),
        lambda: gi.gemm_fp8_impl(a_col, a_col_s, True, g_col, g_col_s, False, torch.bfloat16, True, SG.BLOCKWISE),
    ]
    for run in runs:
        first = run()
        for _ in range(9):
            assert torch.equal(first, run())
    nv.check_status(x.device)


def test_accumulate_into_out(mods):
    qi, gi, nv, SG, _ = mods
    a, b = make((256, 256), torch.bfloat16, 33), make((384, 256), torch.bfloat16, 34)
    qa, sa = qi.quantize_fp8_tensorwise_impl(a, torch.float8_e4m3fn)
    qb, sb = qi.quantize_fp8_tensorwise_impl(b, torch.float8_e4m3fn)
    out = torch.ones(256, 384, dtype=torch.float32, device="cuda")
    gi.gemm_fp8_accum_impl(qa, sa, False, qb, sb, True, out, False, SG.TENSORWISE)
    nv.check_status(out.device)
    ref = _ref(u8(qa), f32(sa), u8(qb), f32(sb), "e4m3", "e4m3") + 1.0
    assert og.rel_frobenius(f32(out), ref) <= 1e-5


@pytest.mark.parametrize("M,N,K", [(128, 256, 128), (256, 512, 384), (255, 520, 576), (1024, 1024, 2048)])
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
def test_blockwise_fwd_dgrad_wgrad(mods, M, N, K, out_dtype):
    """The three GEMMs of the blockwise path (primus_turbo/pytorch/ops/gemm_fp8.py:429-553 of the reference):
    forward NT, dgrad NN against the 128x128-scaled weight, wgrad TN from the column-scaled copies."""
    qi, gi, nv, SG, _ = mods
    f8, f5 = torch.float8_e4m3fn, torch.float8_e5m2
    a = make((M, K), torch.bfloat16, 41, "outlier")
    w = make((N, K), torch.bfloat16, 42, "weight")
    g = make((M, N), torch.bfloat16, 43, "small")
    a_row, a_rs, a_col, a_cs = qi.quant_fp8_blockwise_dual_impl(a, f8)
    w_q, w_s = qi.quant_fp8_blockwise_for_weight_impl(w, f8)
    g_row, g_rs, g_col, g_cs = qi.quant_fp8_blockwise_dual_impl(g, f5)
    tol = FP8_TOL if out_dtype == torch.bfloat16 else 1e-5
    da_row = oq.dequantize_fp8_blockwise(u8(a_row), f32(a_rs), "e4m3", 1)
    da_col = oq.dequantize_fp8_blockwise(u8(a_col), f32(a_cs), "e4m3", 0)
    dw = oq.dequantize_fp8_blockwise_weight(u8(w_q), f32(w_s), "e4m3")
    dg_row = oq.dequantize_fp8_blockwise(u8(g_row), f32(g_rs), "e5m2", 1)
    dg_col = oq.dequantize_fp8_blockwise(u8(g_col), f32(g_cs), "e5m2", 0)
    # forward: [M,K] x [N,K]^T
    c = gi.gemm_fp8_impl(a_row, a_rs, False, w_q, w_s, True, out_dtype, False, SG.BLOCKWISE)
    nv.check_status(c.device)
    assert og.rel_frobenius(f32(c), og.gemm_nt(da_row, dw)) <= tol
    # dgrad: [M,N] x [N,K]
    da = gi.gemm_fp8_impl(g_row, g_rs, False, w_q, w_s, False, out_dtype, False, SG.BLOCKWISE)
    nv.check_status(c.device)
    assert og.rel_frobenius(f32(da), dg_row @ dw) <= tol
    # wgrad: a_col^T [K,M] x g_col [M,N] -> [K,N], returned transposed as [N,K]
    dwg = gi.gemm_fp8_impl(a_col, a_cs, True, g_col, g_cs, False, out_dtype, True, SG.BLOCKWISE)
    nv.check_status(c.device)
    assert dwg.shape == (N, K)
    assert og.rel_frobenius(f32(dwg), (da_col.T @ dg_col).T) <= tol
