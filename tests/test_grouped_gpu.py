"""Grouped quantizers and grouped GEMMs (MoE path) against the CPU oracle and the reference's acceptance gates
(tests/pytorch/ops/test_grouped_gemm_fp8.py of the reference: SNR gates, zero-length groups, zero output tail)."""
import numpy as np
import pytest
import torch

from oracle import gemm as og
from oracle import quant as oq
from tests._util import assert_bits_equal, f32, fmt_of, make, u8

pytestmark = pytest.mark.gpu

LENS = [[100, 0, 128, 29], [1, 300], [0, 0, 5], [256, 256], [130] * 7 + [0]]


def snr(x, ref):
    x, ref = x.float(), ref.float()
    return float(10 * torch.log10(ref.pow(2).sum() / (x - ref).pow(2).sum().clamp_min(1e-30)))


@pytest.fixture(scope="module")
def mods():
    import primus_turbo.pytorch as turbo
    from primus_turbo.pytorch.core.low_precision import (Float8QuantConfig, Format, ScaleDtype, ScalingGranularity,
                                                         ScalingRecipe)
    from primus_turbo.pytorch.kernels import _native as nv
    from primus_turbo.pytorch.kernels.grouped_gemm import grouped_gemm_fp8_impl as ggi
    from primus_turbo.pytorch.kernels.quantization import quantization_impl as qi
    return dict(turbo=turbo, nv=nv, qi=qi, ggi=ggi, SG=ScalingGranularity, SR=ScalingRecipe, Cfg=Float8QuantConfig,
                Format=Format, ScaleDtype=ScaleDtype)


def _offs(lens):
    lens_t = torch.tensor(lens, dtype=torch.int64, device="cuda")
    offs = torch.zeros(len(lens) + 1, dtype=torch.int64, device="cuda")
    offs[1:] = torch.cumsum(lens_t, 0)
    return lens_t, offs


@pytest.mark.parametrize("dtype", [torch.float8_e4m3fn, torch.float8_e5m2, torch.float4_e2m1fn_x2])
@pytest.mark.parametrize("lens", LENS)
def test_grouped_mx_quantize(mods, dtype, lens):
    qi = mods["qi"]
    lens_t, offs = _offs(lens)
    M, N = int(sum(lens)), 96
    x = make((M, N), torch.bfloat16, 51, "outlier")
    fmt = fmt_of(dtype)
    impl = qi.grouped_quantize_mxfp4_impl if fmt == "e2m1" else qi.grouped_quantize_mxfp8_impl
    q_row, s_row, q_col, s_col, lr, orow, lc, ocol = impl(x, dtype, None, 32, lens_t, offs, with_trans=True)
    row_align = 1 if fmt == "e2m1" else 32
    wq_r, ws_r, wl_r, wo_r = oq.quantize_mx_grouped(f32(x), fmt, np.array(lens), 1, row_align=row_align)
    col_align = 256 if fmt == "e2m1" else 128   # fp4: one GEMM stage spans 256 contraction elements
    wq_c, ws_c, wl_c, wo_c = oq.quantize_mx_grouped(f32(x), fmt, np.array(lens), 0, col_align=col_align)
    assert np.array_equal(orow.cpu().numpy(), wo_r) and np.array_equal(ocol.cpu().numpy(), wo_c)
    assert np.array_equal(lr.cpu().numpy(), wl_r) and np.array_equal(lc.cpu().numpy(), wl_c)
    gq_r, gs_r, gq_c, gs_c = u8(q_row), u8(s_row), u8(q_col), u8(s_col)
    for g, n in enumerate(lens):  # only real rows of the row-wise copy are defined
        r0 = int(wo_r[g])
        assert_bits_equal(gs_r[r0:r0 + n], ws_r[r0:r0 + n], f"row scales g{g}")
        assert_bits_equal(gq_r[r0:r0 + n], wq_r[r0:r0 + n], f"row bytes g{g}")
    tot = int(wo_c[-1])
    div = 2 if fmt == "e2m1" else 1
    assert_bits_equal(gs_c[:, :tot // 32], ws_c[:, :tot // 32], "col scales")
    assert_bits_equal(gq_c[:, :tot // div], wq_c[:, :tot // div], "col bytes")
    # single-direction entry points agree with the dual one
    q1, s1, _, o1 = impl(x, dtype, 1, 32, lens_t, offs)
    for g, n in enumerate(lens):
        r0 = int(wo_r[g])
        assert torch.equal(q1.view(torch.uint8)[r0:r0 + n], q_row.view(torch.uint8)[r0:r0 + n])
    q0, s0, _, o0 = impl(x, dtype, 0, 32, lens_t, offs)
    assert torch.equal(q0.view(torch.uint8)[:, :tot // div], q_col.view(torch.uint8)[:, :tot // div])


@pytest.mark.parametrize("lens", LENS)
@pytest.mark.parametrize("trans_b", [True, False])
def test_grouped_blockwise_gemm_and_variable_k(mods, lens, trans_b):
    qi, ggi, nv, SG = mods["qi"], mods["ggi"], mods["nv"], mods["SG"]
    lens_t, offs = _offs(lens)
    G, M, K, N = len(lens), int(sum(lens)), 256, 384
    a = make((M, K), torch.bfloat16, 52, "outlier")
    w = make((G, N, K) if trans_b else (G, K, N), torch.bfloat16, 53, "weight")
    f8 = torch.float8_e4m3fn
    a_row, a_col, a_s_row, a_s_col, plens, poffs = qi.quant_fp8_blockwise_segment_m_row_col_impl(a, f8, 128, lens_t, offs)
    w_q, w_s = qi.quant_fp8_blockwise_for_weight_impl(w, f8)
    out = ggi.grouped_gemm_fp8_impl(a_row, w_q, a_s_row, w_s, lens_t, offs, False, trans_b, torch.float32, SG.BLOCKWISE)
    nv.check_status(out.device)
    da = oq.dequantize_fp8_blockwise(u8(a_row), np.ascontiguousarray(f32(a_s_row).T), "e4m3", 1)
    dw = np.stack([oq.dequantize_fp8_blockwise_weight(u8(w_q)[g], f32(w_s)[g], "e4m3") for g in range(G)])
    dwn = dw if trans_b else dw.transpose(0, 2, 1)
    ref = og.grouped_gemm_nt(da, dwn, np.array(lens))
    if M:
        assert og.rel_frobenius(f32(out), ref) <= 1e-5
    # variable-K wgrad: C[g] = a_col[seg]^T . g_col[seg]
    go = make((M, N), torch.bfloat16, 54, "small")
    g_row, g_col, g_s_row, g_s_col, _, _ = qi.quant_fp8_blockwise_segment_m_row_col_impl(go, torch.float8_e5m2, 128, lens_t, offs)
    wg = ggi.grouped_gemm_fp8_variable_k_impl(a_col, g_col, a_s_col, g_s_col, plens, poffs, True, False, True, torch.float32,
                                              SG.BLOCKWISE)
    nv.check_status(out.device)
    assert wg.shape == (G, N, K)
    mp = int(poffs[-1])
    dac = oq.dequantize_fp8_blockwise(u8(a_col)[:mp], f32(a_s_col)[:mp // 128], "e4m3", 0)
    dgc = oq.dequantize_fp8_blockwise(u8(g_col)[:mp], f32(g_s_col)[:mp // 128], "e5m2", 0)
    refw = og.grouped_gemm_variable_k(dgc, dac, plens.cpu().numpy())
    for g, n in enumerate(lens):
        if n == 0:
            assert float(wg[g].abs().max()) == 0.0      # empty group: exact zeros
    assert og.rel_frobenius(f32(wg), refw) <= 1e-5


@pytest.mark.parametrize("lens", LENS)
def test_grouped_mx_gemm_and_variable_k(mods, lens):
    qi, ggi, nv, SG, SR = mods["qi"], mods["ggi"], mods["nv"], mods["SG"], mods["SR"]
    lens_t, offs = _offs(lens)
    G, M, K, N = len(lens), int(sum(lens)), 256, 320
    a = make((M, K), torch.bfloat16, 55, "outlier")
    w = make((G, N, K), torch.bfloat16, 56, "weight")
    f8 = torch.float8_e4m3fn
    a_row, a_s_row, a_col, a_s_col, _, orow, lcol, ocol = qi.grouped_quantize_mxfp8_impl(a, f8, None, 32, lens_t, offs, with_trans=True)
    two_d = SR(use_2d_block=True)
    w_row, w_s_row, w_col, w_s_col = qi.quantize_mxfp8_impl(w, f8, None, 32, with_trans=True, scaling_recipe=two_d,
                                                            scaling_recipe_for_trans=two_d)
    out = ggi.grouped_gemm_fp8_impl(a_row, w_row, a_s_row, w_s_row, lens_t, orow, False, True, torch.float32, SG.MX_BLOCKWISE,
                                    group_offs_out=offs)
    nv.check_status(out.device)
    orow_h = orow.cpu().numpy()
    da = np.concatenate([oq.dequantize_mx(u8(a_row)[orow_h[g]:orow_h[g] + n], u8(a_s_row)[orow_h[g]:orow_h[g] + n], "e4m3")
                         for g, n in enumerate(lens)] or [np.zeros((0, K), np.float32)])
    dw = np.stack([oq.dequantize_mx(u8(w_row)[g], u8(w_s_row)[g], "e4m3") for g in range(G)])
    ref = og.grouped_gemm_nt(da, dw, np.array(lens))
    if M:
        assert og.rel_frobenius(f32(out)[:M], ref) <= 1e-5
    assert float(out[M:].abs().max() if out.shape[0] > M else 0.0) == 0.0   # rows past the last group stay zero
    # variable-K: C[g] = g_col[:, seg] . a_col[:, seg]^T over the 128-padded segments
    go = make((M, N), torch.bfloat16, 57, "small")
    g_row, g_s_row, g_col, g_s_col, _, _, lcol, ocol = qi.grouped_quantize_mxfp8_impl(go, torch.float8_e5m2, None, 32, lens_t, offs,
                                                                                      with_trans=True)
    wg = ggi.grouped_gemm_fp8_variable_k_impl(g_col, a_col, g_s_col, a_s_col, lcol, ocol, False, False, False, torch.float32,
                                              SG.MX_BLOCKWISE)
    nv.check_status(out.device)
    assert wg.shape == (G, N, K)
    tot = int(ocol[-1])
    dgc = oq.dequantize_mx(u8(g_col)[:, :tot], u8(g_s_col)[:, :tot // 32], "e5m2")     # [N, tot]
    dac = oq.dequantize_mx(u8(a_col)[:, :tot], u8(a_s_col)[:, :tot // 32], "e4m3")     # [K, tot]
    refw = og.grouped_gemm_variable_k(dgc.T, dac.T, lcol.cpu().numpy())
    assert og.rel_frobenius(f32(wg), refw) <= 1e-5


def _cfg(m, gran, fmt):
    SG, Cfg, Format, SD = m["SG"], m["Cfg"], m["Format"], m["ScaleDtype"]
    kw = {}
    if gran == "BLOCKWISE":
        kw["block_size"] = 128
    if gran == "MX_BLOCKWISE":
        kw.update(block_size=32, scale_dtype=SD.E8M0)
    return Cfg(format=Format[fmt], granularity=SG[gran], **kw)


@pytest.mark.parametrize("gran", ["TENSORWISE", "ROWWISE", "BLOCKWISE", "MX_BLOCKWISE"])
@pytest.mark.parametrize("fmt", ["E4M3", "HYBRID"])
@pytest.mark.parametrize("lens", [[128, 256, 64], [100, 0, 300, 29], [512] * 8])
def test_grouped_gemm_fp8_op(mods, gran, fmt, lens):
    turbo = mods["turbo"]
    torch.manual_seed(7)
    lens_t, offs = _offs(lens)
    G, M, K, N = len(lens), int(sum(lens)), 512, 384
    a = torch.randn(M, K, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    b = torch.randn(G, N, K, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    a_ref, b_ref = a.detach().clone().requires_grad_(), b.detach().clone().requires_grad_()
    out = turbo.ops.grouped_gemm_fp8(a, b, lens_t, trans_b=True, config=_cfg(mods, gran, fmt))
    ref = torch.cat([a_ref[offs[g]:offs[g + 1]].float() @ b_ref[g].float().t() for g in range(G)]).to(torch.bfloat16)
    assert out.shape == ref.shape
    go = torch.randn_like(ref)
    out.backward(go)
    ref.backward(go)
    gate_b = 25 if fmt == "E4M3" else 20
    assert snr(out.detach(), ref.detach()) > 25
    assert snr(a.grad, a_ref.grad) > gate_b
    for g, n in enumerate(lens):
        if n == 0:
            assert float(b.grad[g].abs().max()) == 0.0
        elif n >= 64:
            assert snr(b.grad[g], b_ref.grad[g]) > gate_b


@pytest.mark.parametrize("lens", LENS + [[64, 192, 1, 127, 129]])
@pytest.mark.parametrize("C", [64, 200, 4096 + 16])
def test_grouped_transpose_pad_is_exact(mods, lens, C):
    """Token-major -> [features, padded tokens] copy: every group's rows land in its 128-aligned segment, all other
    bytes are zero."""
    qi = mods["qi"]
    lens_t, offs = _offs(lens)
    M, G = int(sum(lens)), len(lens)
    x = torch.randint(0, 256, (M, C), dtype=torch.uint8, device="cuda")
    plens, poffs = qi.compute_padded_group_offs(lens_t, 128)
    y = qi.grouped_transpose_pad(x, offs, poffs)
    T = (M + 127) // 128 * 128 + 128 * G
    assert tuple(y.shape) == (C, T)
    want = torch.zeros((C, T), dtype=torch.uint8, device="cuda")
    po = poffs.cpu().tolist()
    o = offs.cpu().tolist()
    for g, n in enumerate(lens):
        assert po[g] % 128 == 0
        want[:, po[g]:po[g] + n] = x[o[g]:o[g] + n].t()
    assert torch.equal(y, want)


@pytest.mark.parametrize("shape", [(1, 64, 64), (3, 100, 72), (8, 384, 512)])
@pytest.mark.parametrize("dtype", [torch.uint8, torch.bfloat16, torch.float32])
def test_transpose_batched(mods, shape, dtype):
    qi = mods["qi"]
    x = torch.randint(0, 200, shape, device="cuda").to(dtype)
    assert torch.equal(qi.transpose_batched(x), x.transpose(1, 2).contiguous())


@pytest.mark.parametrize("gran", ["TENSORWISE", "ROWWISE"])
@pytest.mark.parametrize("trans_b", [True, False])
@pytest.mark.parametrize("lens", [[100, 0, 300, 29], [512] * 4])
def test_grouped_tensor_row_no_host_sync_and_layouts(mods, gran, trans_b, lens):
    """Tensorwise / rowwise grouped GEMM, both weight layouts, forward and backward with host synchronisation
    forbidden: group lengths are never read on the host."""
    turbo = mods["turbo"]
    torch.manual_seed(11)
    lens_t, offs = _offs(lens)
    G, M, K, N = len(lens), int(sum(lens)), 256, 384
    a = torch.randn(M, K, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    b = torch.randn((G, N, K) if trans_b else (G, K, N), device="cuda", dtype=torch.bfloat16, requires_grad=True)
    a_ref, b_ref = a.detach().clone().requires_grad_(), b.detach().clone().requires_grad_()
    go = torch.randn(M, N, device="cuda", dtype=torch.bfloat16)
    cfg = _cfg(mods, gran, "E4M3")
    torch.cuda.synchronize()
    torch.cuda.set_sync_debug_mode("error")
    try:
        out = turbo.ops.grouped_gemm_fp8(a, b, lens_t, group_offs=offs, trans_b=trans_b, config=cfg)
        out.backward(go)
    finally:
        torch.cuda.set_sync_debug_mode("default")
    o = offs.cpu().tolist()
    ref = torch.cat([a_ref[o[g]:o[g + 1]].float() @ (b_ref[g].float().t() if trans_b else b_ref[g].float())
                     for g in range(G)]).to(torch.bfloat16)
    ref.backward(go)
    assert b.grad.shape == b_ref.grad.shape
    assert snr(out.detach(), ref.detach()) > 25
    assert snr(a.grad, a_ref.grad) > 25
    for g, n in enumerate(lens):
        if n == 0:
            assert float(b.grad[g].abs().max()) == 0.0
        elif n >= 64:
            assert snr(b.grad[g], b_ref.grad[g]) > 25


@pytest.mark.parametrize("gran", ["TENSORWISE", "ROWWISE"])
def test_grouped_tensor_row_fused_main_grad(mods, gran):
    """fuse_bgrad_accum_pattern='megatron': the wgrad is added into b.main_grad in place."""
    turbo = mods["turbo"]
    torch.manual_seed(12)
    lens = [200, 56, 0, 256]
    lens_t, offs = _offs(lens)
    G, M, K, N = len(lens), int(sum(lens)), 256, 128
    a = torch.randn(M, K, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    b = torch.randn(G, N, K, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    go = torch.randn(M, N, device="cuda", dtype=torch.bfloat16)
    cfg = _cfg(mods, gran, "E4M3")
    out = turbo.ops.grouped_gemm_fp8(a, b, lens_t, trans_b=True, config=cfg)
    out.backward(go)
    plain = b.grad.float().clone()
    b2 = b.detach().clone().requires_grad_()
    base = torch.randn(G, N, K, device="cuda", dtype=torch.float32)
    b2.main_grad = base.clone()
    b2.grad_added_to_main_grad = False
    a2 = a.detach().clone().requires_grad_()
    out2 = turbo.ops.grouped_gemm_fp8(a2, b2, lens_t, trans_b=True, config=cfg, fuse_bgrad_accum_pattern="megatron")
    out2.backward(go)
    assert b2.grad_added_to_main_grad
    got = b2.main_grad - base
    assert snr(got, plain) > 40   # same products, fp32 accumulate vs bf16 rounding of the plain path


@pytest.mark.parametrize("dtype", [torch.float8_e4m3fn, torch.float4_e2m1fn_x2])
@pytest.mark.parametrize("lens", [[100, 0, 128, 29], [256, 256]])
def test_grouped_quantized_tensor_roundtrip(mods, dtype, lens):
    """QuantizedTensor.quantize(group_lens=...) produces the grouped payload of the grouped quantizers, and
    dequantize() brings back the tight [total_m, N] tensor."""
    from primus_turbo.pytorch.core.quantized_tensor import QuantizedTensor
    qi, SG = mods["qi"], mods["SG"]
    lens_t, offs = _offs(lens)
    M, N = int(sum(lens)), 160
    x = make((M, N), torch.bfloat16, 52, "normal")
    impl = qi.grouped_quantize_mxfp4_impl if dtype == torch.float4_e2m1fn_x2 else qi.grouped_quantize_mxfp8_impl
    axes = (-1,) if dtype == torch.float4_e2m1fn_x2 else (-1, -2)
    for axis in axes:
        qt = QuantizedTensor.quantize(x, dtype, SG.MX_BLOCKWISE, axis=axis, block_size=32, group_lens=lens_t)
        assert qt.is_grouped_tensor and tuple(qt.shape) == (M, N)
        q, s, plens, poffs = impl(x, dtype, 1 if axis == -1 else 0, 32, lens_t, offs, with_trans=False)
        assert torch.equal(qt.group_offs, poffs) and torch.equal(qt.orig_group_offs, offs)
        back = qt.dequantize()
        assert tuple(back.shape) == (M, N)
        step = 0.25 if dtype == torch.float4_e2m1fn_x2 else 0.0625   # half a mantissa step at the block's top binade, x2
        blk = x.float().abs().amax().item()
        assert float((back.float() - x.float()).abs().max()) <= 2 * step * blk
        # group by group against the dense dequantizer on the same rows
        o = offs.cpu().tolist()
        for g, n in enumerate(lens):
            if n == 0:
                continue
            seg = x[o[g]:o[g] + n].contiguous()
            dense = QuantizedTensor.quantize(seg, dtype, SG.MX_BLOCKWISE, axis=axis, block_size=32).dequantize()
            assert torch.equal(back[o[g]:o[g] + n], dense), f"group {g} axis {axis}"


def test_grouped_mx_gemm_prequantized_operands(mods):
    """grouped_gemm_fp8 (MX) with QuantizedTensor inputs: the forward is bit-identical to the path that quantizes
    inside the operator; backward passes the same gates."""
    from primus_turbo.pytorch.core.quantized_tensor import QuantizedTensor
    turbo, SG, SR = mods["turbo"], mods["SG"], mods["SR"]
    torch.manual_seed(5)
    lens = [200, 0, 312, 128]
    lens_t, offs = _offs(lens)
    G, M, K, N = len(lens), int(sum(lens)), 256, 384
    a = torch.randn(M, K, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    b = torch.randn(G, N, K, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    cfg = _cfg(mods, "MX_BLOCKWISE", "E4M3")
    plain = turbo.ops.grouped_gemm_fp8(a, b, lens_t, trans_b=True, config=cfg)
    a_q = QuantizedTensor.quantize(a.detach(), torch.float8_e4m3fn, SG.MX_BLOCKWISE, axis=-1, block_size=32, group_lens=lens_t)
    b_q = QuantizedTensor.quantize(b.detach(), torch.float8_e4m3fn, SG.MX_BLOCKWISE, axis=-1, block_size=32,
                                   scaling_recipe=SR(use_2d_block=True))
    a_q.requires_grad_()
    b_q.requires_grad_()
    out = turbo.ops.grouped_gemm_fp8(a_q, b_q, lens_t, trans_b=True, config=cfg)
    assert torch.equal(out, plain)
    go = torch.randn_like(out)
    out.backward(go)
    o = offs.cpu().tolist()
    a_ref, b_ref = a.detach().clone().requires_grad_(), b.detach().clone().requires_grad_()
    ref = torch.cat([a_ref[o[g]:o[g + 1]].float() @ b_ref[g].float().t() for g in range(G)]).to(torch.bfloat16)
    ref.backward(go)
    assert snr(a_q.grad, a_ref.grad) > 20
    for g, n in enumerate(lens):
        if n >= 64:
            assert snr(b_q.grad[g], b_ref.grad[g]) > 20
