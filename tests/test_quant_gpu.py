"""Bit-exact parity of the CUDA quantizers (called through the C ABI) with the CPU oracle."""
import numpy as np
import pytest
import torch

from oracle import quant as oq
from tests._util import assert_bits_equal, f32, fmt_of, make, u8

pytestmark = pytest.mark.gpu

FP8 = [torch.float8_e4m3fn, torch.float8_e5m2]
SRC = [torch.bfloat16, torch.float16, torch.float32]


@pytest.fixture(scope="module")
def qi():
    from primus_turbo.pytorch.kernels.quantization import quantization_impl
    return quantization_impl


@pytest.mark.parametrize("dtype", FP8)
@pytest.mark.parametrize("src", SRC)
@pytest.mark.parametrize("shape", [(1, 15), (16, 17), (333, 2881), (1024, 4096)])
def test_tensorwise(qi, dtype, src, shape):
    x = make(shape, src, 11, "outlier")
    q, s = qi.quantize_fp8_tensorwise_impl(x, dtype)
    wq, ws = oq.quantize_fp8_tensorwise(f32(x), fmt_of(dtype))
    assert_bits_equal(f32(s), ws, "scale_inv")
    assert_bits_equal(u8(q), wq, "bytes")


def test_tensorwise_misaligned_matches_aligned(qi):
    # tests/pytorch/ops/test_quantization.py:91-100 of the reference: the unaligned fallback must give identical bytes
    base = make((4096 * 33 + 1,), torch.bfloat16, 5)
    x_mis = base[1:]
    x_al = x_mis.clone()
    q1, s1 = qi.quantize_fp8_tensorwise_impl(x_mis, torch.float8_e4m3fn)
    q2, s2 = qi.quantize_fp8_tensorwise_impl(x_al, torch.float8_e4m3fn)
    assert torch.equal(q1.view(torch.uint8), q2.view(torch.uint8)) and torch.equal(s1, s2)


def test_tensorwise_amax_spike(qi):
    # test_quantization.py:103-130: one planted spike must set the scale wherever it sits
    for pos in (0, 12345, 8 * 1024 * 1024 - 1):
        x = torch.full((8 * 1024 * 1024,), 0.5, dtype=torch.bfloat16, device="cuda")
        x[pos] = 1000.0
        _, s = qi.quantize_fp8_tensorwise_impl(x, torch.float8_e4m3fn)
        assert abs(float(s) - 1000.0 / 448.0) < 1e-4


def test_tensorwise_given_scale(qi):
    x = make((257, 130), torch.bfloat16, 3)
    scale = torch.tensor(37.5, device="cuda")
    q, s = qi.quantize_fp8_tensorwise_impl(x, torch.float8_e4m3fn, scale)
    want = oq._quant_clamp_encode(f32(x), np.float32(37.5), "e4m3")
    assert_bits_equal(u8(q), want)
    assert float(s) == float(np.float32(1.0) / np.float32(37.5))


@pytest.mark.parametrize("dtype", FP8)
@pytest.mark.parametrize("src", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("shape,axis", [((5, 2881), -1), ((64, 256), -1), ((3, 65, 136), -1), ((3, 65, 136), 1),
                                        ((130, 257), 0), ((2048, 4096), 0), ((2048, 4096), 1), ((2, 3, 40), 0)])
def test_rowwise(qi, dtype, src, shape, axis):
    x = make(shape, src, 12, "outlier")
    q, s = qi.quantize_fp8_rowwise_impl(x, dtype, axis)
    wq, ws = oq.quantize_fp8_rowwise(f32(x), fmt_of(dtype), axis)
    assert_bits_equal(f32(s), ws, "scale_inv")
    assert_bits_equal(u8(q), wq, "bytes")


@pytest.mark.parametrize("dtype", FP8)
def test_dequantize_tensor_row(qi, dtype):
    x = make((130, 264), torch.bfloat16, 4)
    q, s = qi.quantize_fp8_tensorwise_impl(x, dtype)
    y = qi.dequantize_fp8_tensorwise_impl(q, torch.float32, s)
    assert_bits_equal(f32(y), oq.dequantize_fp8(u8(q), f32(s), fmt_of(dtype)))
    for axis in (0, 1):
        q, s = qi.quantize_fp8_rowwise_impl(x, dtype, axis)
        y = qi.dequantize_fp8_rowwise_impl(q, torch.float32, axis, s)
        assert_bits_equal(f32(y), oq.dequantize_fp8(u8(q), f32(s), fmt_of(dtype)))
        assert torch.allclose(y, x.float(), rtol=1e-1, atol=1e-1)


@pytest.mark.parametrize("dtype", FP8)
@pytest.mark.parametrize("src", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("shape", [(128, 128), (200, 384), (257, 130), (1, 7), (1024, 2048)])
def test_blockwise(qi, dtype, src, shape):
    x = make(shape, src, 13, "outlier")
    fmt = fmt_of(dtype)
    for axis in (0, 1):
        q, s = qi.quant_fp8_blockwise_impl(x, dtype, axis)
        wq, ws = oq.quantize_fp8_blockwise(f32(x), fmt, axis)
        assert_bits_equal(f32(s), ws, f"scale axis{axis}")
        assert_bits_equal(u8(q), wq, f"bytes axis{axis}")
        y = qi.dequant_fp8_blockwise_impl(q, s, torch.float32, axis)
        assert_bits_equal(f32(y), oq.dequantize_fp8_blockwise(wq, ws, fmt, axis), "dequant")
    qr, sr, qc, sc = qi.quant_fp8_blockwise_dual_impl(x, dtype)
    wqr, wsr, wqc, wsc = oq.quantize_fp8_blockwise_dual(f32(x), fmt)
    for got, want, name in ((u8(qr), wqr, "q_row"), (f32(sr), wsr, "s_row"), (u8(qc), wqc, "q_col"), (f32(sc), wsc, "s_col")):
        assert_bits_equal(got, want, name)


@pytest.mark.parametrize("dtype", FP8)
@pytest.mark.parametrize("shape", [(256, 384), (3, 200, 130), (2, 128, 128)])
def test_blockwise_weight(qi, dtype, shape):
    w = make(shape, torch.bfloat16, 14, "weight")
    q, s = qi.quant_fp8_blockwise_for_weight_impl(w, dtype)
    wq, ws = oq.quantize_fp8_blockwise_weight(f32(w), fmt_of(dtype))
    assert_bits_equal(f32(s), ws, "scales")
    assert_bits_equal(u8(q), wq, "bytes")
    y = qi.dequant_fp8_blockwise_for_weight_impl(q, s, torch.float32)
    assert_bits_equal(f32(y), oq.dequantize_fp8_blockwise_weight(wq, ws, fmt_of(dtype)))


@pytest.mark.parametrize("dtype", FP8)
@pytest.mark.parametrize("lens", [[100, 0, 128, 29], [1, 300], [0, 0, 5], [256, 256], [130] * 7 + [0]])
def test_blockwise_segment_m(qi, dtype, lens):
    lens_t = torch.tensor(lens, dtype=torch.int64, device="cuda")
    offs = torch.zeros(len(lens) + 1, dtype=torch.int64, device="cuda")
    offs[1:] = torch.cumsum(lens_t, 0)
    M, N = int(sum(lens)), 264
    x = make((M, N), torch.bfloat16, 15, "outlier")
    x_row, x_col, s_row, s_col, plens, poffs = qi.quant_fp8_blockwise_segment_m_row_col_impl(x, dtype, 128, lens_t, offs)
    w_row, w_col, ws_row, ws_col, wpl, wpo = oq.quantize_fp8_blockwise_segment_m(f32(x), fmt_of(dtype), np.array(lens))
    assert np.array_equal(plens.cpu().numpy(), wpl) and np.array_equal(poffs.cpu().numpy(), wpo)
    mp = int(wpo[-1])
    assert_bits_equal(u8(x_row), w_row, "row bytes")
    assert_bits_equal(f32(s_row), ws_row, "row scales")
    assert_bits_equal(u8(x_col)[:mp], w_col[:mp], "col bytes")
    assert_bits_equal(f32(s_col)[:mp // 128], ws_col[:mp // 128], "col scales")


def test_group_offs(qi):
    from primus_turbo.pytorch.kernels import _native as nv
    for G in (1, 7, 256, 1500):
        lens = torch.randint(0, 1000, (G,), dtype=torch.int64, device="cuda")
        offs = torch.empty(G + 1, dtype=torch.int64, device="cuda")
        nv.check(nv.lib().pt_compute_group_offs(nv.ptr(lens), G, nv.ptr(offs), nv.stream()))
        want = torch.zeros(G + 1, dtype=torch.int64, device="cuda")
        want[1:] = torch.cumsum(lens, 0)
        assert torch.equal(offs, want)
        plens, poffs = qi.compute_padded_group_offs(lens, 128)
        wl = (lens + 127) // 128 * 128
        assert torch.equal(plens, wl) and torch.equal(poffs[1:], torch.cumsum(wl, 0))


@pytest.mark.parametrize("shape", [(64, 64), (130, 257), (1, 5), (1000, 3)])
@pytest.mark.parametrize("dtype", [torch.uint8, torch.bfloat16, torch.float32])
def test_transpose(qi, shape, dtype):
    x = torch.randint(0, 255, shape, device="cuda").to(dtype)
    assert torch.equal(qi.transpose_2d(x), x.t().contiguous())


MXF = [torch.float8_e4m3fn, torch.float8_e5m2, torch.float4_e2m1fn_x2]


@pytest.mark.parametrize("dtype", MXF)
@pytest.mark.parametrize("src", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("shape", [(128, 128), (200, 96), (1, 32), (257, 416), (1024, 2048)])
@pytest.mark.parametrize("use_2d", [False, True])
def test_mx_single_and_dual(qi, dtype, src, shape, use_2d):
    from primus_turbo.pytorch.core.low_precision import ScalingRecipe
    x = make(shape, src, 16, "outlier")
    fmt = fmt_of(dtype)
    rec = ScalingRecipe(use_2d_block=use_2d)
    impl = qi.quantize_mxfp4_impl if fmt == "e2m1" else qi.quantize_mxfp8_impl
    want = {ax: oq.quantize_mx(f32(x), fmt, ax, use_2d) for ax in (0, 1)}
    for ax in (0, 1):
        q, s = impl(x, dtype, ax, 32, scaling_recipe=rec)
        assert_bits_equal(u8(s), want[ax][1], f"scale axis{ax}")
        assert_bits_equal(u8(q), want[ax][0], f"bytes axis{ax}")
    qr, sr, qc, sc = impl(x, dtype, None, 32, with_trans=True, scaling_recipe=rec, scaling_recipe_for_trans=rec)
    for got, w, name in ((u8(sr), want[1][1], "s_row"), (u8(qr), want[1][0], "q_row"), (u8(sc), want[0][1], "s_col"),
                         (u8(qc), want[0][0], "q_col")):
        assert_bits_equal(got, w, name)


@pytest.mark.parametrize("dtype", MXF)
def test_mx_batched_and_round_trip(qi, dtype):
    x = make((3, 200, 96), torch.bfloat16, 17)
    fmt = fmt_of(dtype)
    impl = qi.quantize_mxfp4_impl if fmt == "e2m1" else qi.quantize_mxfp8_impl
    deq = qi.dequantize_mxfp4_impl if fmt == "e2m1" else qi.dequantize_mxfp8_impl
    tol = 0.5 if fmt == "e2m1" else 1e-1
    for ax in (1, 2):
        q, s = impl(x, dtype, ax, 32)
        wq, ws = oq.quantize_mx_batched(f32(x), fmt, ax)
        assert_bits_equal(u8(s), ws, "scales")
        assert_bits_equal(u8(q), wq, "bytes")
        y = deq(q, torch.float32, ax, 32, s, orig_shape=x.shape)
        assert y.shape == x.shape
        assert torch.allclose(y, x.float(), rtol=tol, atol=tol)


@pytest.mark.parametrize("rht_row,rht_col", [(True, False), (False, True), (True, True)])
def test_mxfp4_rht(qi, rht_row, rht_col):
    from primus_turbo.pytorch.core.low_precision import ScalingRecipe
    x = make((200, 160), torch.bfloat16, 18)
    qr, sr, qc, sc = qi.quantize_mxfp4_impl(x, torch.float4_e2m1fn_x2, None, 32, with_trans=True,
                                            scaling_recipe=ScalingRecipe(use_rht=rht_row),
                                            scaling_recipe_for_trans=ScalingRecipe(use_rht=rht_col))
    wqr, wsr = oq.quantize_mx(f32(x), "e2m1", 1, False, rht_row)
    wqc, wsc = oq.quantize_mx(f32(x), "e2m1", 0, False, rht_col)
    assert_bits_equal(u8(sr), wsr, "s_row"); assert_bits_equal(u8(qr), wqr, "q_row")
    assert_bits_equal(u8(sc), wsc, "s_col"); assert_bits_equal(u8(qc), wqc, "q_col")


def test_errors_are_reported(qi):
    x = make((64, 48), torch.bfloat16, 1)
    with pytest.raises(RuntimeError, match="divisible by 32"):
        qi.quantize_mxfp8_impl(x, torch.float8_e4m3fn, 1, 32)
    with pytest.raises(RuntimeError, match="CUDA tensors only"):
        qi.quantize_fp8_tensorwise_impl(x.cpu(), torch.float8_e4m3fn)


@pytest.mark.parametrize("dtype", FP8)
def test_nan_and_inf_inputs_follow_the_reference_clamp(qi, dtype):
    """A NaN element takes no part in the amax and leaves through the reference's clamp: fmax(fmin(NaN, qmax), -qmax) =
    +qmax for tensorwise / rowwise / blockwise (device/quant_utils.cuh:33-40), fmin(fmax(NaN, -lim), lim) = -qmax for MX
    (quantization_mxfp8.cu:131-136); +-inf saturate to +-qmax.  Bytes and scales equal the oracle's, which applies the
    same two clamps."""
    fmt = fmt_of(dtype)
    x = make((256, 256), torch.bfloat16, 21, "normal")
    x[3, 5] = float("nan")
    x[200, 17] = float("nan")
    xf = f32(x)
    for name, got, want in [
        ("tensorwise", qi.quantize_fp8_tensorwise_impl(x, dtype), oq.quantize_fp8_tensorwise(xf, fmt)),
        ("rowwise", qi.quantize_fp8_rowwise_impl(x, dtype, -1), oq.quantize_fp8_rowwise(xf, fmt, -1)),
        ("colwise", qi.quantize_fp8_rowwise_impl(x, dtype, -2), oq.quantize_fp8_rowwise(xf, fmt, -2)),
        ("blockwise row", qi.quant_fp8_blockwise_impl(x, dtype, 1), oq.quantize_fp8_blockwise(xf, fmt, 1)),
        ("blockwise col", qi.quant_fp8_blockwise_impl(x, dtype, 0), oq.quantize_fp8_blockwise(xf, fmt, 0)),
        ("mx row", qi.quantize_mxfp8_impl(x, dtype, 1, 32), oq.quantize_mx(xf, fmt, 1)),
        ("mx col", qi.quantize_mxfp8_impl(x, dtype, 0, 32), oq.quantize_mx(xf, fmt, 0)),
    ]:
        assert_bits_equal(u8(got[0]), want[0], name + " bytes")
        if name.startswith("mx"):
            assert_bits_equal(u8(got[1]), want[1], name + " scales")
        else:
            np.testing.assert_array_equal(f32(got[1]).reshape(-1), np.asarray(want[1], dtype=np.float32).reshape(-1), err_msg=name)
    qmax_code = {"e4m3": 0x7E, "e5m2": 0x7B}[fmt]
    assert int(u8(qi.quantize_fp8_rowwise_impl(x, dtype, -1)[0])[3, 5]) == qmax_code          # NaN -> +qmax
    assert int(u8(qi.quantize_mxfp8_impl(x, dtype, 1, 32)[0])[3, 5]) == (qmax_code | 0x80)    # NaN -> -qmax (MX)
    # dual outputs see the same NaN handling in both copies
    qr, sr, qc, sc = qi.quantize_mxfp8_impl(x, dtype, None, 32, with_trans=True)
    assert_bits_equal(u8(qr), oq.quantize_mx(xf, fmt, 1)[0], "mx dual row bytes")
    assert_bits_equal(u8(qc), oq.quantize_mx(xf, fmt, 0)[0], "mx dual col bytes")
    # +-inf: the block's amax is inf (scale byte from the exponent field 255), the elements saturate
    y = make((128, 128), torch.bfloat16, 22, "normal")
    y[1, 2] = float("inf")
    y[70, 90] = float("-inf")
    got = qi.quantize_fp8_rowwise_impl(y, dtype, -1)
    want = oq.quantize_fp8_rowwise(f32(y), fmt, -1)
    assert_bits_equal(u8(got[0]), want[0], "rowwise bytes with inf")
    got = qi.quantize_mxfp8_impl(y, dtype, 1, 32)
    want = oq.quantize_mx(f32(y), fmt, 1)
    assert_bits_equal(u8(got[0]), want[0], "mx bytes with inf")
    assert_bits_equal(u8(got[1]), want[1], "mx scales with inf")


def test_mx_row_copy_at_a_16_byte_aligned_output(qi):
    """The row copy is written with 32-byte stores when its address allows and with 16-byte ones otherwise: an output
    buffer that is only 16-byte aligned must receive the same bytes."""
    from primus_turbo.pytorch.kernels import _native as nv
    M, N = 256, 384
    x = make((M, N), torch.bfloat16, 23, "normal")
    q_ref, s_ref = qi.quantize_mxfp8_impl(x, torch.float8_e4m3fn, 1, 32)
    raw = torch.zeros(M * N + 64, dtype=torch.uint8, device="cuda")
    q_view = raw[16:16 + M * N]
    assert q_view.data_ptr() % 32 == 16
    s_row = torch.empty((M, N // 32), dtype=torch.uint8, device="cuda")
    nv.check(nv.lib().pt_quantize_mx(nv.ptr(x), nv.src_code(x.dtype), 1, M, N, nv.fmt_code(torch.float8_e4m3fn), nv.PT_MX_ROW,
                                      q_view.data_ptr(), nv.ptr(s_row), None, None, nv.stream(x.device)), "quantize_mx")
    torch.cuda.synchronize()
    assert torch.equal(q_view.view(M, N), q_ref.view(torch.uint8))
    assert torch.equal(s_row, s_ref.view(torch.uint8))
    assert int(raw[:16].max()) == 0 and int(raw[16 + M * N:].max()) == 0


@pytest.mark.gpu
@pytest.mark.parametrize("which", ["mxfp8_dual", "mxfp4_dual", "mxfp8_dual_2d", "blockwise_dual", "rowwise", "tensorwise"])
def test_quantizers_give_the_same_bytes_every_launch(which):
    """Twenty launches on an input that fills every SM several times over must agree byte for byte with the first: the
    warp-specialised quantizers synchronise their warp groups with mbarriers and named barriers, and a lost or early
    hand-over shows up as a few blocks that differ in a few launches of a hundred, not as a wrong result every time."""
    import primus_turbo.pytorch as turbo
    from primus_turbo.pytorch.core.low_precision import ScalingGranularity as SG, ScalingRecipe
    from primus_turbo.pytorch.kernels.quantization import quantization_impl as qi
    g = torch.Generator(device="cuda").manual_seed(77)
    x = torch.randn(4096, 7168, device="cuda", dtype=torch.bfloat16, generator=g)
    f8, f4 = torch.float8_e4m3fn, torch.float4_e2m1fn_x2
    run = {
        "mxfp8_dual": lambda: qi.quantize_mxfp8_impl(x, f8, None, 32, True),
        "mxfp4_dual": lambda: qi.quantize_mxfp4_impl(x, f4, None, 32, True),
        "mxfp8_dual_2d": lambda: qi.quantize_mxfp8_impl(x, f8, None, 32, True, ScalingRecipe(use_2d_block=True), ScalingRecipe(use_2d_block=True)),
        "blockwise_dual": lambda: qi.quant_fp8_blockwise_dual_impl(x, f8),
        "rowwise": lambda: qi.quantize_fp8_rowwise_impl(x, f8, -1) + qi.quantize_fp8_rowwise_impl(x, f8, -2),
        "tensorwise": lambda: qi.quantize_fp8_tensorwise_impl(x, f8),
    }[which]
    bits = lambda t: t.view(torch.uint8) if t.element_size() == 1 else t.view(torch.int32)
    first = [bits(t).clone() for t in run()]
    for _ in range(20):
        for a, b in zip(run(), first):
            assert torch.equal(bits(a), b)
