"""Gated activations with probabilities and RMSNorm: the CUDA kernels against the numpy oracle and against torch's own
operators, over the shapes and types of the reference's tests/pytorch/ops/test_activation.py and test_normalization.py."""
import numpy as np
import pytest
import torch
import torch.nn.functional as F

from oracle import activation_norm as O

pytestmark = pytest.mark.gpu

TOL = {torch.float32: dict(rtol=1e-4, atol=1e-4), torch.float16: dict(rtol=1e-2, atol=1e-2), torch.bfloat16: dict(rtol=1e-2, atol=1e-2)}
# against the fp64 oracle: one rounding of the output type plus the hardware exp / divide approximations
ULP = {torch.float32: 2e-6, torch.float16: 1.0e-3, torch.bfloat16: 8.0e-3}


def _ops():
    from primus_turbo.pytorch.ops import geglu_with_probs, rmsnorm, rmsnorm_residual, swiglu_with_probs
    return swiglu_with_probs, geglu_with_probs, rmsnorm, rmsnorm_residual


def _close_to_oracle(got, want, dtype, scale=1.0):
    got = got.detach().double().cpu().numpy()
    err = np.abs(got - want)
    bound = ULP[dtype] * scale * np.maximum(np.abs(want), 1e-3 if dtype != torch.float32 else 1e-6) + (1e-6 if dtype == torch.float32 else 1e-4)
    bad = err > bound
    assert not bad.any(), f"{bad.sum()} of {bad.size} outside the bound; worst {err.max()} at want {want.flat[np.argmax(err)]}"


@pytest.mark.parametrize("act", ["silu", "gelu"])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16, torch.float32])
@pytest.mark.parametrize("shape", [(1, 1, 128), (1, 128, 256), (8, 2025, 128), (1, 2048, 2048), (2, 513, 7168)])
@pytest.mark.parametrize("masked", [False, True])
def test_glu_with_probs(act, dtype, shape, masked):
    swiglu, geglu, _, _ = _ops()
    func = swiglu if act == "silu" else geglu
    b, s, h = shape
    g = torch.Generator(device="cuda").manual_seed(b * 131 + s + h)
    x = torch.randn(b, s, 2 * h, device="cuda", dtype=dtype, generator=g).requires_grad_()
    probs = torch.rand(b, s, device="cuda", dtype=torch.float32, generator=g).requires_grad_()
    row_mask = None
    if masked:
        row_mask = torch.zeros(b * s, device="cuda", dtype=torch.int64)
        row_mask[: max(1, (b * s * 3) // 4)] = 1
    out = func(x, probs, row_mask)
    assert out.shape == (b * s, h) and out.dtype == dtype
    xf = x.detach().float().view(b * s, 2 * h).cpu().numpy()
    pf = probs.detach().view(-1).cpu().numpy()
    mk = None if row_mask is None else row_mask.cpu().numpy()
    _close_to_oracle(out, O.glu_fwd(xf, pf, act, mk), dtype)

    # torch's operators, the reference's own check
    xr = x.detach().clone().view(b * s, 2 * h).requires_grad_()
    pr = probs.detach().clone().view(-1, 1).requires_grad_()
    a, bb = torch.chunk(xr.float(), 2, dim=-1)
    ref = ((F.silu(a) if act == "silu" else F.gelu(a)) * bb * pr).to(dtype)
    live = slice(None) if row_mask is None else row_mask.bool()
    torch.testing.assert_close(out[live], ref[live], **TOL[dtype])

    grad = torch.randn(b * s, h, device="cuda", dtype=dtype, generator=g)   # not ones: exercises the full derivative
    out.backward(grad)
    gx, gp = O.glu_bwd(grad.float().cpu().numpy(), xf, pf, act, mk)
    _close_to_oracle(x.grad.view(b * s, 2 * h), gx, dtype, scale=2.0)
    got_gp = probs.grad.view(-1).double().cpu().numpy()
    tol_gp = (2e-3 if dtype != torch.float32 else 1e-4) * (np.abs(gx).max() + 1) * np.sqrt(h) + 1e-3
    assert np.abs(got_gp - gp).max() <= tol_gp
    ref.backward(grad)
    if row_mask is None:
        torch.testing.assert_close(x.grad.view_as(xr.grad), xr.grad, **TOL[dtype])
        torch.testing.assert_close(probs.grad.view(-1), pr.grad.view(-1), rtol=2e-2 if dtype != torch.float32 else 1e-3, atol=0.1 if dtype != torch.float32 else 1e-3)
    else:
        dead = ~row_mask.bool()
        assert (out[dead] == 0).all() and (x.grad.view(b * s, -1)[dead] == 0).all() and (probs.grad.view(-1)[dead] == 0).all()


def test_glu_rejects_bad_arguments():
    swiglu, _, _, _ = _ops()
    x = torch.randn(4, 256, device="cuda", dtype=torch.bfloat16)
    with pytest.raises(AssertionError):
        swiglu(x, torch.rand(4, device="cuda", dtype=torch.bfloat16), None)          # probs must be fp32
    with pytest.raises(AssertionError):
        swiglu(x, torch.rand(3, device="cuda"), None)                                # rows differ
    with pytest.raises(AssertionError):
        swiglu(x, torch.rand(4, device="cuda"), torch.ones(4, device="cuda", dtype=torch.int32))   # mask must be int64
    assert swiglu(torch.empty(0, 256, device="cuda", dtype=torch.bfloat16), torch.empty(0, device="cuda"), None).shape == (0, 128)


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
@pytest.mark.parametrize("outer", [(1,), (511,), (4096,), (2, 300)])
@pytest.mark.parametrize("H", [33, 128, 513, 4096, 5120, 7168, 8192, 16384])
@pytest.mark.parametrize("zero_centered", [False, True])
def test_rmsnorm(dtype, outer, H, zero_centered):
    if zero_centered and H not in (128, 4096, 8192):
        pytest.skip("zero-centred gain: the reference's three widths")
    _, _, rmsnorm, _ = _ops()
    eps = 1e-6
    g = torch.Generator(device="cuda").manual_seed(H + len(outer))
    x = torch.randn(*outer, H, device="cuda", dtype=dtype, generator=g).requires_grad_()
    gamma = (torch.randn(H, device="cuda", dtype=dtype, generator=g) * (0.1 if zero_centered else 1.0)).requires_grad_()
    y = rmsnorm(x, gamma, eps, zero_centered)
    assert y.shape == x.shape and y.dtype == dtype
    xf, gf = x.detach().float().view(-1, H).cpu().numpy(), gamma.detach().float().cpu().numpy()
    want, _ = O.rmsnorm_fwd(xf, gf, eps, zero_centered)
    _close_to_oracle(y.view(-1, H), want, dtype)
    xr, gr = x.detach().clone().requires_grad_(), gamma.detach().clone().requires_grad_()
    w_eff = (gr.float() + 1.0).to(dtype) if zero_centered else gr
    y_ref = F.rms_norm(xr, [H], w_eff, eps)
    torch.testing.assert_close(y, y_ref, **TOL[dtype])
    grad = torch.randn(*outer, H, device="cuda", dtype=dtype, generator=g)
    y.backward(grad)
    y_ref.backward(grad)
    dx, dg = O.rmsnorm_bwd(grad.float().view(-1, H).cpu().numpy(), xf, gf, eps, zero_centered)
    _close_to_oracle(x.grad.view(-1, H), dx, dtype, scale=4.0)
    rows = xf.shape[0]
    dg_tol = (1e-5 if dtype == torch.float32 else 4e-3) * (np.abs(dg) + np.sqrt(rows)) + 1e-4
    assert (np.abs(gamma.grad.double().cpu().numpy() - dg) <= dg_tol).all()
    torch.testing.assert_close(x.grad, xr.grad, **TOL[dtype])


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
@pytest.mark.parametrize("rows,H", [(1, 128), (511, 4096), (1024, 8192), (77, 520), (64, 12288)])
def test_rmsnorm_residual(dtype, rows, H):
    _, _, _, rmsnorm_residual = _ops()
    eps = 1e-5
    g = torch.Generator(device="cuda").manual_seed(rows + H)
    x = torch.randn(rows, H, device="cuda", dtype=dtype, generator=g).requires_grad_()
    r = torch.randn(rows, H, device="cuda", dtype=dtype, generator=g).requires_grad_()
    gamma = torch.randn(H, device="cuda", dtype=dtype, generator=g).requires_grad_()
    y, xpr = rmsnorm_residual(x, r, gamma, eps)
    assert torch.equal(xpr, (x.detach().float() + r.detach().float()).to(dtype))   # the sum is rounded once, to the tensor's type
    want, _ = O.rmsnorm_fwd(xpr.detach().float().cpu().numpy(), gamma.detach().float().cpu().numpy(), eps)
    _close_to_oracle(y, want, dtype)
    gy = torch.randn(rows, H, device="cuda", dtype=dtype, generator=g)
    gx = torch.randn(rows, H, device="cuda", dtype=dtype, generator=g)
    torch.autograd.backward([y, xpr], [gy, gx])
    dx, dg = O.rmsnorm_bwd(gy.float().cpu().numpy(), xpr.detach().float().cpu().numpy(), gamma.detach().float().cpu().numpy(), eps,
                           dxpr=gx.float().cpu().numpy())
    _close_to_oracle(x.grad, dx, dtype, scale=4.0)
    assert torch.equal(x.grad, r.grad)
    dg_tol = (1e-5 if dtype == torch.float32 else 4e-3) * (np.abs(dg) + np.sqrt(rows)) + 1e-4
    assert (np.abs(gamma.grad.double().cpu().numpy() - dg) <= dg_tol).all()


def test_rmsnorm_statistics_alone():
    from primus_turbo.pytorch.kernels.normalization.rmsnorm_impl import rmsnorm_stats_impl
    x = torch.randn(300, 4096, device="cuda", dtype=torch.bfloat16)
    rstd = rmsnorm_stats_impl(x, 1e-6)
    want = torch.rsqrt(x.float().pow(2).mean(-1) + 1e-6)
    torch.testing.assert_close(rstd, want, rtol=1e-5, atol=1e-6)


# ----------------------------------------------------------------------------------- operator + MX quantizer in one pass
def _same(a, b):
    for u, v in zip(a, b):
        if isinstance(u, torch.Tensor) and u.dtype != torch.float32 and u.dtype != torch.int64:
            assert torch.equal(u.view(torch.uint8), v.view(torch.uint8))
        else:
            assert torch.equal(u, v)


@pytest.mark.parametrize("act", ["silu", "gelu"])
@pytest.mark.parametrize("out_dtype", [torch.float8_e4m3fn, torch.float4_e2m1fn_x2])
@pytest.mark.parametrize("rows,H,masked", [(128, 64, False), (1000, 1408, True), (4096, 2048, False), (77, 7168, False)])
def test_glu_quantize_mx_fused_equals_two_kernels(act, out_dtype, rows, H, masked):
    from primus_turbo.pytorch.kernels.quantization.quantization_impl import glu_quantize_mx_impl
    g = torch.Generator(device="cuda").manual_seed(rows + H)
    x = torch.randn(rows, 2 * H, device="cuda", dtype=torch.bfloat16, generator=g) * 3
    x[rows // 2, :7] = float("nan")
    x[0, 40:72] = 0
    probs = torch.rand(rows, device="cuda", generator=g)
    mask = None
    if masked:
        mask = (torch.rand(rows, device="cuda", generator=g) > 0.2).to(torch.int64)
    fused = glu_quantize_mx_impl(x, probs, mask, act, out_dtype, fused=True)
    plain = glu_quantize_mx_impl(x, probs, mask, act, out_dtype, fused=False)
    _same(fused, plain)
    assert glu_quantize_mx_impl(x, probs, mask, act, out_dtype)[0].shape == plain[0].shape   # the default picks the fused kernel here


@pytest.mark.parametrize("act", ["silu", "gelu"])
@pytest.mark.parametrize("out_dtype", [torch.float8_e4m3fn, torch.float4_e2m1fn_x2])
@pytest.mark.parametrize("lens", [[128, 256, 128], [1, 0, 300, 77, 129], [0, 0, 5], [640] * 4 + [0] * 3 + [33]])
def test_grouped_glu_quantize_mx_fused_equals_two_kernels(act, out_dtype, lens):
    from primus_turbo.pytorch.kernels.quantization.quantization_impl import grouped_glu_quantize_mx_impl
    H = 512
    rows = sum(lens)
    g = torch.Generator(device="cuda").manual_seed(rows)
    x = torch.randn(rows, 2 * H, device="cuda", dtype=torch.bfloat16, generator=g)
    probs = torch.rand(rows, device="cuda", generator=g)
    gl = torch.tensor(lens, device="cuda", dtype=torch.int64)
    go = torch.cat([gl.new_zeros(1), gl.cumsum(0)])
    fused = grouped_glu_quantize_mx_impl(x, probs, None, act, out_dtype, gl, go, fused=True)
    plain = grouped_glu_quantize_mx_impl(x, probs, None, act, out_dtype, gl, go, fused=False)
    # the buffers are allocated past the last group's padded end; compare what the groups cover
    q_row_f, s_row_f, q_col_f, s_col_f, lr, orow, lc, ocol = fused
    q_row_p, s_row_p, q_col_p, s_col_p = plain[:4]
    assert torch.equal(orow, plain[5]) and torch.equal(ocol, plain[7])
    fp4 = out_dtype == torch.float4_e2m1fn_x2
    for i, n in enumerate(lens):
        r0 = int(orow[i])
        assert torch.equal(q_row_f.view(torch.uint8)[r0:r0 + n], q_row_p.view(torch.uint8)[r0:r0 + n])
        assert torch.equal(s_row_f.view(torch.uint8)[r0:r0 + n], s_row_p.view(torch.uint8)[r0:r0 + n])
        c0, c1 = int(ocol[i]), int(ocol[i + 1])
        d = 2 if fp4 else 1
        assert torch.equal(q_col_f.view(torch.uint8)[:, c0 // d:c1 // d], q_col_p.view(torch.uint8)[:, c0 // d:c1 // d])
        assert torch.equal(s_col_f.view(torch.uint8)[:, c0 // 32:c1 // 32], s_col_p.view(torch.uint8)[:, c0 // 32:c1 // 32])


@pytest.mark.parametrize("out_dtype", [torch.float8_e4m3fn, torch.float4_e2m1fn_x2])
@pytest.mark.parametrize("rows,H,zc", [(128, 128, False), (1000, 4096, True), (4096, 7168, False), (300, 8192 + 32, False)])
def test_rmsnorm_quantize_mx_fused_equals_two_kernels(out_dtype, rows, H, zc):
    from primus_turbo.pytorch.kernels.quantization.quantization_impl import rmsnorm_quantize_mx_impl
    g = torch.Generator(device="cuda").manual_seed(rows + H)
    x = torch.randn(rows, H, device="cuda", dtype=torch.bfloat16, generator=g) * 2
    gamma = torch.randn(H, device="cuda", dtype=torch.bfloat16, generator=g)
    fused = rmsnorm_quantize_mx_impl(x, gamma, 1e-6, zc, out_dtype, fused=True)
    plain = rmsnorm_quantize_mx_impl(x, gamma, 1e-6, zc, out_dtype, fused=False)
    _same(fused, plain)


def test_fused_quantizer_refuses_what_it_does_not_cover():
    from primus_turbo.pytorch.kernels.quantization.quantization_impl import fused_mx_supported, glu_quantize_mx_impl
    x16 = torch.randn(64, 256, device="cuda", dtype=torch.float16)
    assert not fused_mx_supported(x16, 128, torch.float8_e4m3fn, True)
    assert not fused_mx_supported(x16.bfloat16(), 96, torch.float8_e4m3fn, True)
    with pytest.raises(RuntimeError):   # forced onto the one-pass kernel: the library says no, it does not compute something else
        glu_quantize_mx_impl(x16, torch.rand(64, device="cuda"), None, "silu", torch.float8_e4m3fn, fused=True)
    out = glu_quantize_mx_impl(x16, torch.rand(64, device="cuda"), None, "silu", torch.float8_e4m3fn)   # two kernels
    assert out[0].shape == (64, 128)


@pytest.mark.parametrize("act", ["silu", "gelu"])
def test_glu_quantize_mxfp4_with_hadamard_columns_fused_equals_two_kernels(act):
    """The MXFP4 recipe's operand layout (row-wise copy plain, transposed copy after the 16-point Hadamard transform),
    dense and grouped."""
    from primus_turbo.pytorch.kernels.quantization.quantization_impl import glu_quantize_mx_impl, grouped_glu_quantize_mx_impl
    F4 = torch.float4_e2m1fn_x2
    g = torch.Generator(device="cuda").manual_seed(5)
    rows, H = 1280, 1024
    x = torch.randn(rows, 2 * H, device="cuda", dtype=torch.bfloat16, generator=g)
    probs = torch.rand(rows, device="cuda", generator=g)
    _same(glu_quantize_mx_impl(x, probs, None, act, F4, fused=True, col_rht=True), glu_quantize_mx_impl(x, probs, None, act, F4, fused=False, col_rht=True))
    assert not torch.equal(glu_quantize_mx_impl(x, probs, None, act, F4, col_rht=True)[2].view(torch.uint8),
                           glu_quantize_mx_impl(x, probs, None, act, F4)[2].view(torch.uint8))   # the transform is applied
    lens = [256, 0, 512, 256, 256]
    gl = torch.tensor(lens, device="cuda", dtype=torch.int64)
    go = torch.cat([gl.new_zeros(1), gl.cumsum(0)])
    f = grouped_glu_quantize_mx_impl(x, probs, None, act, F4, gl, go, fused=True, col_rht=True)
    u = grouped_glu_quantize_mx_impl(x, probs, None, act, F4, gl, go, fused=False, col_rht=True)
    ocol = f[7]
    for i, n in enumerate(lens):
        c0, c1 = int(ocol[i]), int(ocol[i + 1])
        assert torch.equal(f[0].view(torch.uint8)[sum(lens[:i]):sum(lens[:i + 1])], u[0].view(torch.uint8)[sum(lens[:i]):sum(lens[:i + 1])])
        assert torch.equal(f[2].view(torch.uint8)[:, c0 // 2:c1 // 2], u[2].view(torch.uint8)[:, c0 // 2:c1 // 2])
        assert torch.equal(f[3].view(torch.uint8)[:, c0 // 32:c1 // 32], u[3].view(torch.uint8)[:, c0 // 32:c1 // 32])


@pytest.mark.parametrize("out_dtype", [torch.float8_e4m3fn, torch.float4_e2m1fn_x2])
def test_fused_rmsnorm_quantizer_gives_the_same_bytes_every_launch(out_dtype):
    """Thirty launches on an input of 3584 tiles (three CTAs per SM, every warp role busy) must all write the bytes of the
    two-kernel path: a barrier between the in-place normalisation and the row / column passes that lets one warp through
    early shows up here as a handful of blocks quantized from half-normalised data in a few launches of a hundred."""
    from primus_turbo.pytorch.kernels.quantization.quantization_impl import rmsnorm_quantize_mx_impl
    rows, H = 4096, 7168
    g = torch.Generator(device="cuda").manual_seed(rows + H)
    x = torch.randn(rows, H, device="cuda", dtype=torch.bfloat16, generator=g) * 2
    gamma = torch.randn(H, device="cuda", dtype=torch.bfloat16, generator=g)
    plain = rmsnorm_quantize_mx_impl(x, gamma, 1e-6, False, out_dtype, fused=False)
    for _ in range(30):
        _same(rmsnorm_quantize_mx_impl(x, gamma, 1e-6, False, out_dtype, fused=True), plain)


@pytest.mark.parametrize("out_dtype", [torch.float8_e4m3fn, torch.float8_e5m2, torch.float4_e2m1fn_x2])
@pytest.mark.parametrize("rows,H,zc", [(1, 32, False), (128, 128, False), (1000, 4096, True), (333, 7168, False), (64, 8192, False), (50, 160, True)])
def test_rmsnorm_row_quantizer_one_pass_equals_two_kernels(out_dtype, rows, H, zc):
    """Forward-only form: RMSNorm and the row-wise MX copy in one pass write the bytes of RMSNorm kernel + quantizer, and
    the same rstd; a NaN and an all-zero row included."""
    from primus_turbo.pytorch.kernels.quantization.quantization_impl import rmsnorm_quantize_mx_row_impl
    g = torch.Generator(device="cuda").manual_seed(rows * 7 + H)
    x = torch.randn(rows, H, device="cuda", dtype=torch.bfloat16, generator=g) * 3
    if rows > 2:
        x[1] = 0
        x[2, H // 2] = float("nan")
    if rows > 4:
        x[3, 5] = float("inf")          # rstd = 0: one NaN (inf * 0) in a row of zeros, so a single block holds a NaN
    gamma = torch.randn(H, device="cuda", dtype=torch.bfloat16, generator=g)
    if H > 64:
        gamma[40] = float("nan")        # a NaN gain: one NaN per row, in one block only
    one = rmsnorm_quantize_mx_row_impl(x, gamma, 1e-6, zc, out_dtype, fused=True)
    two = rmsnorm_quantize_mx_row_impl(x, gamma, 1e-6, zc, out_dtype, fused=False)
    assert torch.equal(one[0].view(torch.uint8), two[0].view(torch.uint8))
    assert torch.equal(one[1].view(torch.uint8), two[1].view(torch.uint8))
    assert torch.equal(one[2].view(torch.int32), two[2].view(torch.int32))


@pytest.mark.parametrize("act", ["silu", "gelu"])
@pytest.mark.parametrize("out_dtype", [torch.float8_e4m3fn, torch.float8_e5m2, torch.float4_e2m1fn_x2])
@pytest.mark.parametrize("rows,H,masked", [(1, 32, False), (128, 64, False), (1000, 1408, True), (300, 2048, False), (77, 7168, False), (50, 2080, True)])
def test_glu_row_quantizer_one_pass_equals_two_kernels(act, out_dtype, rows, H, masked):
    """Forward-only form: gated activation and the row-wise MX copy in one pass write the bytes of activation kernel +
    quantizer; masked rows, a NaN and an inf included."""
    from primus_turbo.pytorch.kernels.quantization.quantization_impl import glu_quantize_mx_row_impl
    g = torch.Generator(device="cuda").manual_seed(rows * 3 + H)
    x = torch.randn(rows, 2 * H, device="cuda", dtype=torch.bfloat16, generator=g) * 2
    if rows > 2:
        x[1, 3] = float("nan")
        x[2, H + 7] = float("inf")
    probs = torch.rand(rows, device="cuda", generator=g)
    mask = (torch.rand(rows, device="cuda", generator=g) > 0.3).to(torch.int64) if masked else None
    one = glu_quantize_mx_row_impl(x, probs, mask, act, out_dtype, fused=True)
    two = glu_quantize_mx_row_impl(x, probs, mask, act, out_dtype, fused=False)
    assert torch.equal(one[0].view(torch.uint8), two[0].view(torch.uint8))
    assert torch.equal(one[1].view(torch.uint8), two[1].view(torch.uint8))
