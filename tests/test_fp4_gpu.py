"""MXFP4 GEMMs (tcgen05 kind::mxf4.block_scale): against the fp32 matmul of the dequantized operands (stated tolerance:
relative Frobenius error <= 5e-2; with fp32 output the only difference is summation order) and the reference's SNR
gates against the unquantized product: > 10 dB dense (tests/pytorch/ops/test_gemm_fp4.py:120), > 8 dB grouped
(tests/pytorch/ops/test_grouped_gemm_fp4.py:55-57)."""
import numpy as np
import pytest
import torch

from oracle import gemm as og
from oracle import quant as oq
from tests._util import f32, make, u8

pytestmark = pytest.mark.gpu
F4 = torch.float4_e2m1fn_x2


def snr(x, ref):
    x, ref = x.float(), ref.float()
    return float(10 * torch.log10(ref.pow(2).sum() / (x - ref).pow(2).sum().clamp_min(1e-30)))


@pytest.fixture(scope="module")
def m():
    import primus_turbo.pytorch as turbo
    from primus_turbo.pytorch.core.low_precision import ScalingRecipe
    from primus_turbo.pytorch.kernels import _native as nv
    from primus_turbo.pytorch.kernels.gemm import gemm_fp4_impl as g4
    from primus_turbo.pytorch.kernels.grouped_gemm import grouped_gemm_fp4_impl as gg4
    from primus_turbo.pytorch.kernels.quantization import quantization_impl as qi
    return dict(turbo=turbo, nv=nv, g4=g4, gg4=gg4, qi=qi, SR=ScalingRecipe)


@pytest.mark.parametrize("M,N,K", [(128, 128, 256), (256, 512, 384), (255, 520, 576), (1024, 2048, 1024), (512, 240, 128)])
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_gemm_fp4_dense(m, M, N, K, out_dtype):
    qi, g4, nv, SR = m["qi"], m["g4"], m["nv"], m["SR"]
    a, b = make((M, K), torch.bfloat16, 61, "outlier"), make((N, K), torch.bfloat16, 62, "weight")
    qa, sa = qi.quantize_mxfp4_impl(a, F4, 1, 32)
    qb, sb = qi.quantize_mxfp4_impl(b, F4, 1, 32, scaling_recipe=SR(use_2d_block=True))
    c = g4.gemm_fp4_impl(qa, sa, False, qb, sb, True, out_dtype, False)
    nv.check_status(c.device)
    ref = og.gemm_nt(oq.dequantize_mx(u8(qa), u8(sa), "e2m1"), oq.dequantize_mx(u8(qb), u8(sb), "e2m1"))
    err = og.rel_frobenius(f32(c), ref)
    assert err <= (1e-5 if out_dtype == torch.float32 else 5e-2), err
    assert og.snr_db(f32(c), f32(a) @ f32(b).T) > 10


def test_gemm_fp4_accumulate_and_transposed_output(m):
    qi, g4, nv = m["qi"], m["g4"], m["nv"]
    a, b = make((256, 256), torch.bfloat16, 63), make((384, 256), torch.bfloat16, 64)
    qa, sa = qi.quantize_mxfp4_impl(a, F4, 1, 32)
    qb, sb = qi.quantize_mxfp4_impl(b, F4, 1, 32)
    ref = og.gemm_nt(oq.dequantize_mx(u8(qa), u8(sa), "e2m1"), oq.dequantize_mx(u8(qb), u8(sb), "e2m1"))
    out = torch.ones(256, 384, dtype=torch.float32, device="cuda")
    g4.gemm_fp4_accum_impl(qa, sa, False, qb, sb, True, out, False)
    ct = g4.gemm_fp4_impl(qa, sa, False, qb, sb, True, torch.float32, True)
    nv.check_status(out.device)
    assert og.rel_frobenius(f32(out), ref + 1.0) <= 1e-5
    assert og.rel_frobenius(f32(ct), ref.T) <= 1e-5


@pytest.mark.parametrize("M,N,K", [(256, 512, 256), (512, 2048, 1024), (255, 512, 576)])
def test_gemm_fp4_op_fwd_bwd(m, M, N, K):
    turbo = m["turbo"]
    torch.manual_seed(5)
    a = torch.randn(M, K, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    b = torch.randn(N, K, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    a_ref, b_ref = a.detach().clone().requires_grad_(), b.detach().clone().requires_grad_()
    out = turbo.ops.gemm_fp4(a, b, trans_b=True)
    ref = a_ref @ b_ref.t()
    g = torch.randn_like(ref)
    out.backward(g)
    ref.backward(g)
    assert snr(out.detach(), ref.detach()) > 10
    assert snr(a.grad, a_ref.grad) > 10
    assert snr(b.grad, b_ref.grad) > 10


@pytest.mark.parametrize("lens", [[128, 256, 64], [100, 0, 300, 29], [512] * 8])
def test_grouped_gemm_fp4_kernels(m, lens):
    qi, gg4, nv, SR = m["qi"], m["gg4"], m["nv"], m["SR"]
    lens_t = torch.tensor(lens, dtype=torch.int64, device="cuda")
    offs = torch.zeros(len(lens) + 1, dtype=torch.int64, device="cuda")
    offs[1:] = torch.cumsum(lens_t, 0)
    G, M, K, N = len(lens), int(sum(lens)), 256, 320
    a = make((M, K), torch.bfloat16, 65, "outlier")
    w = make((G, N, K), torch.bfloat16, 66, "weight")
    a_row, a_s_row, a_col, a_s_col, _, orow, lcol, ocol = qi.grouped_quantize_mxfp4_impl(a, F4, None, 32, lens_t, offs, with_trans=True)
    w_row, w_s_row = qi.quantize_mxfp4_impl(w, F4, 2, 32, scaling_recipe=SR(use_2d_block=True))
    out = gg4.grouped_gemm_fp4_impl(a_row, w_row, a_s_row, w_s_row, lens_t, orow, out_dtype=torch.float32, group_offs_out=offs)
    nv.check_status(out.device)
    da = oq.dequantize_mx(u8(a_row), u8(a_s_row), "e2m1")
    dw = np.stack([oq.dequantize_mx(u8(w_row)[g], u8(w_s_row)[g], "e2m1") for g in range(G)])
    assert og.rel_frobenius(f32(out), og.grouped_gemm_nt(da, dw, np.array(lens))) <= 1e-5
    # variable-K over the 256-padded token segments
    go = make((M, N), torch.bfloat16, 67)
    g_row, g_s_row, g_col, g_s_col, _, _, lcol, ocol = qi.grouped_quantize_mxfp4_impl(go, F4, None, 32, lens_t, offs, with_trans=True)
    wg = gg4.grouped_gemm_fp4_variable_k_impl(g_col, a_col, g_s_col, a_s_col, lcol, ocol, torch.float32)
    nv.check_status(out.device)
    tot = int(ocol[-1])
    dgc = oq.dequantize_mx(u8(g_col)[:, :tot // 2], u8(g_s_col)[:, :tot // 32], "e2m1")
    dac = oq.dequantize_mx(u8(a_col)[:, :tot // 2], u8(a_s_col)[:, :tot // 32], "e2m1")
    refw = og.grouped_gemm_variable_k(dgc.T, dac.T, lcol.cpu().numpy())
    assert wg.shape == (G, N, K)
    assert og.rel_frobenius(f32(wg), refw) <= 1e-5


@pytest.mark.parametrize("lens", [[128, 256, 64], [100, 0, 300, 29], [512] * 8])
def test_grouped_gemm_fp4_op(m, lens):
    turbo = m["turbo"]
    torch.manual_seed(6)
    lens_t = torch.tensor(lens, dtype=torch.int64, device="cuda")
    offs = [0] + list(np.cumsum(lens))
    G, M, K, N = len(lens), int(sum(lens)), 512, 384
    a = torch.randn(M, K, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    b = torch.randn(G, N, K, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    a_ref, b_ref = a.detach().clone().requires_grad_(), b.detach().clone().requires_grad_()
    out = turbo.ops.grouped_gemm_fp4(a, b, lens_t, trans_b=True)
    ref = torch.cat([a_ref[offs[g]:offs[g + 1]].float() @ b_ref[g].float().t() for g in range(G)]).to(torch.bfloat16)
    go = torch.randn_like(ref)
    out.backward(go)
    ref.backward(go)
    assert snr(out.detach(), ref.detach()) > 8
    assert snr(a.grad, a_ref.grad) > 8
    for g, n in enumerate(lens):
        if n == 0:
            assert float(b.grad[g].abs().max()) == 0.0
        elif n >= 64:
            assert snr(b.grad[g], b_ref.grad[g]) > 8


def test_grouped_gemm_fp4_prequantized_operands(m):
    """grouped_gemm_fp4 with QuantizedTensor inputs: same forward bits as quantizing inside the operator; the
    column-wise copies for backward are rebuilt from the dequantized values."""
    from primus_turbo.pytorch.core.low_precision import ScalingGranularity, ScalingRecipe
    from primus_turbo.pytorch.core.quantized_tensor import QuantizedTensor
    turbo = m["turbo"]
    torch.manual_seed(8)
    lens = [200, 0, 312, 128]
    lens_t = torch.tensor(lens, dtype=torch.int64, device="cuda")
    offs = [0] + list(np.cumsum(lens))
    G, M, K, N = len(lens), int(sum(lens)), 256, 384
    a = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    b = torch.randn(G, N, K, device="cuda", dtype=torch.bfloat16)
    plain = turbo.ops.grouped_gemm_fp4(a, b, lens_t, trans_b=True)
    a_q = QuantizedTensor.quantize(a, torch.float4_e2m1fn_x2, ScalingGranularity.MX_BLOCKWISE, axis=-1, block_size=32,
                                   scaling_recipe=ScalingRecipe(), group_lens=lens_t).requires_grad_()
    b_q = QuantizedTensor.quantize(b, torch.float4_e2m1fn_x2, ScalingGranularity.MX_BLOCKWISE, axis=-1, block_size=32,
                                   scaling_recipe=ScalingRecipe(use_2d_block=True)).requires_grad_()
    out = turbo.ops.grouped_gemm_fp4(a_q, b_q, lens_t, trans_b=True)
    assert torch.equal(out, plain)
    go = torch.randn_like(out)
    out.backward(go)
    a_ref, b_ref = a.clone().requires_grad_(), b.clone().requires_grad_()
    ref = torch.cat([a_ref[offs[g]:offs[g + 1]].float() @ b_ref[g].float().t() for g in range(G)]).to(torch.bfloat16)
    ref.backward(go)
    assert snr(a_q.grad, a_ref.grad) > 6
    for g, n in enumerate(lens):
        if n >= 64:
            assert snr(b_q.grad[g], b_ref.grad[g]) > 6


# ------------------------------------------------------------------------------------------------ stochastic rounding
E2M1_GRID = np.array([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0], dtype=np.float32)


def _sr_input():
    """[512, 256] bf16: every 32-block along either axis holds a 6.0 (so its scale is 1.0 and the codes are the values
    themselves) and values that lie between two e2m1 codes."""
    vals = torch.tensor([0.75, 2.25, -3.5, 5.0, 1.25, -0.25, 0.5, 4.0], dtype=torch.float32)
    x = vals.repeat(512, 32)
    x[:, ::32] = 6.0
    x[::32, :] = 6.0
    return x.to(torch.bfloat16).cuda()


@pytest.mark.parametrize("axis", [1, 0])
def test_mxfp4_sr_two_calls_differ_and_stay_between_neighbouring_codes(m, axis):
    """The reference's own SR test (tests/pytorch/ops/test_quantization.py:766-797): two calls on one input differ.
    Added: every result is one of the two codes that bracket the value, exactly representable values never move, and
    the scales are those of round-to-nearest (rounding mode does not touch the scale)."""
    qi, SR = m["qi"], m["SR"]
    x = _sr_input()
    q1, s1 = qi.quantize_mxfp4_impl(x, F4, axis, 32, scaling_recipe=SR(use_sr=True))
    q2, s2 = qi.quantize_mxfp4_impl(x, F4, axis, 32, scaling_recipe=SR(use_sr=True))
    q0, s0 = qi.quantize_mxfp4_impl(x, F4, axis, 32)
    assert not torch.equal(q1.view(torch.uint8), q2.view(torch.uint8))
    assert torch.equal(s1.view(torch.uint8), s0.view(torch.uint8)) and torch.equal(s2.view(torch.uint8), s0.view(torch.uint8))
    xf = f32(x) if axis == 1 else f32(x).T
    for q in (q1, q2):
        d = oq.dequantize_mx(u8(q), u8(s0), "e2m1")[:, : xf.shape[1]]
        lo = np.sign(xf) * E2M1_GRID[np.searchsorted(E2M1_GRID, np.abs(xf), side="right") - 1]
        hi = np.sign(xf) * E2M1_GRID[np.minimum(np.searchsorted(E2M1_GRID, np.abs(xf), side="left"), 7)]
        assert np.all((d == lo) | (d == hi)), "a stochastically rounded value left the two codes around it"
        exact = np.isin(np.abs(xf), E2M1_GRID)
        assert np.array_equal(d[exact], xf[exact])


def test_mxfp4_sr_is_unbiased(m):
    """Mean of the dequantized values over 16 x 512 x 28 draws per value: within 4 standard errors of the value."""
    qi, SR = m["qi"], m["SR"]
    x = _sr_input()
    xf = f32(x)
    acc = np.zeros_like(xf, dtype=np.float64)
    n = 16
    for _ in range(n):
        q, s = qi.quantize_mxfp4_impl(x, F4, 1, 32, scaling_recipe=SR(use_sr=True))
        acc += oq.dequantize_mx(u8(q), u8(s), "e2m1")
    mean = acc / n
    for v in (0.75, 2.25, -3.5, 5.0, 1.25, -0.25):
        sel = xf == np.float32(v)
        lo = E2M1_GRID[np.searchsorted(E2M1_GRID, abs(v), side="right") - 1]
        hi = E2M1_GRID[np.searchsorted(E2M1_GRID, abs(v), side="left")]
        p = (abs(v) - lo) / (hi - lo)
        sigma = (hi - lo) * np.sqrt(p * (1 - p) / (n * sel.sum()))
        assert abs(mean[sel].mean() - v) <= 4 * sigma + 1e-6, (v, mean[sel].mean(), sigma)


def test_mxfp4_sr_dual_and_grouped_and_rht(m):
    """SR through the dual, the Hadamard and the grouped paths: outputs differ between calls, scales do not; the
    round-trip error stays within one code spacing of the (transformed) values."""
    qi, SR = m["qi"], m["SR"]
    x = make((384, 256), torch.bfloat16, 71, "normal")
    sr, sr_rht = SR(use_sr=True), SR(use_sr=True, use_rht=True)
    a = qi.quantize_mxfp4_impl(x, F4, None, 32, with_trans=True, scaling_recipe=sr, scaling_recipe_for_trans=sr_rht)
    b = qi.quantize_mxfp4_impl(x, F4, None, 32, with_trans=True, scaling_recipe=sr, scaling_recipe_for_trans=sr_rht)
    ref = qi.quantize_mxfp4_impl(x, F4, None, 32, with_trans=True, scaling_recipe=SR(), scaling_recipe_for_trans=SR(use_rht=True))
    for i in (0, 2):
        assert not torch.equal(a[i].view(torch.uint8), b[i].view(torch.uint8))
        assert torch.equal(a[i + 1].view(torch.uint8), ref[i + 1].view(torch.uint8))
    d = oq.dequantize_mx(u8(a[0]), u8(a[1]), "e2m1")[:, :256]
    assert og.snr_db(d, f32(x)) > 8
    lens = torch.tensor([100, 0, 156, 128], dtype=torch.int64, device="cuda")
    offs = torch.zeros(5, dtype=torch.int64, device="cuda")
    offs[1:] = torch.cumsum(lens, 0)
    g1 = qi.grouped_quantize_mxfp4_impl(x, F4, None, 32, lens, offs, with_trans=True, scaling_recipe=sr, scaling_recipe_for_trans=sr_rht)
    g2 = qi.grouped_quantize_mxfp4_impl(x, F4, None, 32, lens, offs, with_trans=True, scaling_recipe=sr, scaling_recipe_for_trans=sr_rht)
    assert not torch.equal(g1[0].view(torch.uint8), g2[0].view(torch.uint8))
    assert torch.equal(g1[1].view(torch.uint8), g2[1].view(torch.uint8))


def test_gemm_fp4_with_gradient_sr_passes_the_snr_gate(m):
    turbo = m["turbo"]
    from primus_turbo.pytorch.core.low_precision import Float4QuantConfig
    torch.manual_seed(6)
    cfg = Float4QuantConfig(use_gradient_sr=True)
    a = torch.randn(512, 1024, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    b = torch.randn(768, 1024, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    a_ref, b_ref = a.detach().clone().requires_grad_(), b.detach().clone().requires_grad_()
    g = torch.randn(512, 768, device="cuda", dtype=torch.bfloat16)
    out = turbo.ops.gemm_fp4(a, b, trans_b=True, config=cfg)
    out.backward(g)
    (a_ref @ b_ref.t()).backward(g)
    ga1 = a.grad.clone()
    assert snr(a.grad, a_ref.grad) > 8 and snr(b.grad, b_ref.grad) > 8
    a.grad = b.grad = None
    turbo.ops.gemm_fp4(a, b, trans_b=True, config=cfg).backward(g)
    assert not torch.equal(a.grad, ga1), "gradients under stochastic rounding should differ between runs"
    # grouped
    lens = torch.tensor([200, 0, 312], dtype=torch.int64, device="cuda")
    w = torch.randn(3, 256, 1024, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    x = torch.randn(512, 1024, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    y = turbo.ops.grouped_gemm_fp4(x, w, lens, trans_b=True, config=cfg)
    y.backward(torch.randn_like(y))
    assert torch.isfinite(x.grad.float()).all() and torch.isfinite(w.grad.float()).all()
