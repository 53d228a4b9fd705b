"""Full-size checks at the benchmark shapes (M=8192, N=14336, K=4096 and the MoE grouped shape), where the numpy
oracle cannot restate the whole problem in seconds.  Each test uses a property that does not depend on the size:

* row / column sampling — a 1-D block quantization of a row depends on that row only, and one output element of a
  GEMM on one row of A and one row of B, so sampled rows / columns are compared with the oracle bit for bit
  (quantizers) or to the stated tolerance (GEMMs);
* power-of-two covariance — scaling the input by 2^k leaves MX data bytes unchanged and adds k to every scale byte;
* permutation equivariance and determinism of the GEMM (bit exact);
* round trip — dequantize(quantize(x)) stays within the format's rounding / saturation bound relative to the block amax.
"""
import numpy as np
import pytest
import torch

from oracle import gemm as og
from oracle import quant as oq
from tests._util import assert_bits_equal, f32, make, u8

pytestmark = pytest.mark.gpu

M, N, K = 8192, 14336, 4096
F8 = torch.float8_e4m3fn


@pytest.fixture(scope="module")
def mods():
    from primus_turbo.pytorch.core.low_precision import ScalingGranularity, ScalingRecipe
    from primus_turbo.pytorch.kernels import _native as nv
    from primus_turbo.pytorch.kernels.gemm import gemm_fp8_impl as gi
    from primus_turbo.pytorch.kernels.quantization import quantization_impl as qi
    return qi, gi, nv, ScalingGranularity, ScalingRecipe


@pytest.fixture(scope="module")
def operands():
    a = make((M, K), torch.bfloat16, 101, "outlier")
    w = make((N, K), torch.bfloat16, 102, "weight")
    return a, w


def _rows(n, count, seed):
    return np.sort(np.random.default_rng(seed).choice(n, size=count, replace=False))


def test_mx_quantize_sampled_rows_and_columns(mods, operands):
    qi = mods[0]
    a, _ = operands
    q_row, s_row, q_col, s_col = qi.quantize_mxfp8_impl(a, F8, None, 32, with_trans=True)
    rows = _rows(M, 48, 1)
    want_q, want_s = oq.quantize_mx(f32(a[rows]), "e4m3", 1)
    assert_bits_equal(u8(q_row[rows]), want_q, "row-wise bytes of sampled rows")
    assert_bits_equal(u8(s_row[rows]), want_s, "row-wise scales of sampled rows")
    # the column-wise copy is the transpose [K, M]: row c of it depends on column c of the input only
    cols = _rows(K, 64, 2)  # the oracle wants a multiple of 32 columns
    want_q, want_s = oq.quantize_mx(f32(a[:, cols]), "e4m3", 0)
    assert_bits_equal(u8(q_col[cols]), want_q, "column-wise bytes of sampled columns")
    assert_bits_equal(u8(s_col[cols]), want_s, "column-wise scales of sampled columns")


def test_mx_power_of_two_covariance(mods, operands):
    qi = mods[0]
    a, _ = operands
    q0, s0 = qi.quantize_mxfp8_impl(a, F8, 1, 32)
    q1, s1 = qi.quantize_mxfp8_impl(a * 8, F8, 1, 32)   # exact in bf16: exponents are far from the limits
    assert torch.equal(q0.view(torch.uint8), q1.view(torch.uint8))
    d = s1.view(torch.uint8).to(torch.int32) - s0.view(torch.uint8).to(torch.int32)
    live = s0.view(torch.uint8) != 0  # all-zero blocks keep scale byte 0
    assert bool((d[live] == 3).all()) and bool((d[~live] == 0).all())


def test_mx_round_trip_bound(mods, operands):
    qi = mods[0]
    a, _ = operands
    q, s = qi.quantize_mxfp8_impl(a, F8, 1, 32)
    y = qi.dequantize_mxfp8_impl(q, torch.float32, 1, 32, s, orig_shape=a.shape)
    x = a.float()
    blk_amax = x.abs().view(M, K // 32, 32).amax(-1, keepdim=True).expand(M, K // 32, 32).reshape(M, K)
    # e4m3 keeps 3 mantissa bits: rounding costs at most 2^-4 of the element's binade; the block maximum itself may lie
    # between 448 and 512 scale units (the scale exponent is floor(log2(amax)) - 8) and then saturates: at most 2^-3
    assert bool(((y - x).abs() <= blk_amax * 2.0 ** -3 + 1e-30).all())
    assert og.snr_db(y.cpu().numpy(), x.cpu().numpy()) > 25


@pytest.mark.parametrize("mode", ["row", "col", "weight"])
def test_blockwise_quantize_sampled_blocks(mods, operands, mode):
    qi = mods[0]
    a, w = operands
    if mode == "row":
        q, s = qi.quant_fp8_blockwise_impl(a, F8, 1)
        rows = _rows(M, 32, 3)
        want_q, want_s = oq.quantize_fp8_blockwise(f32(a[rows]), "e4m3", 1)
        assert_bits_equal(u8(q[rows]), want_q, "row-wise bytes")
        assert_bits_equal(f32(s[rows]), want_s, "row-wise scales")
    elif mode == "col":
        q, s = qi.quant_fp8_blockwise_impl(a, F8, 0)
        blocks = _rows(M // 128, 4, 4)  # a 128 x 1 column block lives inside one band of 128 rows
        for b in blocks:
            want_q, want_s = oq.quantize_fp8_blockwise(f32(a[b * 128:(b + 1) * 128]), "e4m3", 0)
            assert_bits_equal(u8(q[b * 128:(b + 1) * 128]), want_q, f"column-wise bytes of band {b}")
            assert_bits_equal(f32(s[b:b + 1]), want_s, f"column-wise scales of band {b}")
    else:
        q, s = qi.quant_fp8_blockwise_for_weight_impl(w, F8)
        blocks = _rows(N // 128, 4, 5)
        for b in blocks:
            want_q, want_s = oq.quantize_fp8_blockwise_weight(f32(w[b * 128:(b + 1) * 128]), "e4m3")
            assert_bits_equal(u8(q[b * 128:(b + 1) * 128]), want_q, f"weight bytes of band {b}")
            assert_bits_equal(f32(s[b:b + 1]), want_s, f"weight scales of band {b}")


@pytest.mark.parametrize("gran", ["tensorwise", "rowwise", "mx", "blockwise"])
def test_gemm_sampled_outputs_determinism_and_permutation(mods, operands, gran):
    qi, gi, nv, SG, SR = mods
    a, w = operands
    rows, cols = _rows(M, 64, 6), _rows(N, 64, 7)
    if gran == "tensorwise":
        (qa, sa), (qw, sw), g = qi.quantize_fp8_tensorwise_impl(a, F8), qi.quantize_fp8_tensorwise_impl(w, F8), SG.TENSORWISE
        a_deq = lambda r: oq.dequantize_fp8(u8(qa[r]), f32(sa), "e4m3")
        w_deq = lambda c: oq.dequantize_fp8(u8(qw[c]), f32(sw), "e4m3")
    elif gran == "rowwise":
        (qa, sa), (qw, sw), g = qi.quantize_fp8_rowwise_impl(a, F8, -1), qi.quantize_fp8_rowwise_impl(w, F8, -1), SG.ROWWISE
        a_deq = lambda r: oq.dequantize_fp8(u8(qa[r]), f32(sa[r]), "e4m3")
        w_deq = lambda c: oq.dequantize_fp8(u8(qw[c]), f32(sw[c]), "e4m3")
    elif gran == "mx":
        (qa, sa), g = qi.quantize_mxfp8_impl(a, F8, 1, 32), SG.MX_BLOCKWISE
        qw, sw = qi.quantize_mxfp8_impl(w, F8, 1, 32, scaling_recipe=SR(use_2d_block=True))
        a_deq = lambda r: oq.dequantize_mx(u8(qa[r]), u8(sa[r]), "e4m3")
        w_deq = lambda c: oq.dequantize_mx(u8(qw[c]), u8(sw[c]), "e4m3")
    else:
        (qa, sa), (qw, sw), g = qi.quant_fp8_blockwise_impl(a, F8, 1), qi.quant_fp8_blockwise_for_weight_impl(w, F8), SG.BLOCKWISE
        a_deq = lambda r: oq.dequantize_fp8_blockwise(u8(qa[r]), f32(sa[r]), "e4m3", 1)
    run = lambda x, sx: gi.gemm_fp8_impl(x, sx, False, qw, sw, True, torch.bfloat16, False, g)
    c = run(qa, sa)
    nv.check_status(c.device)
    if gran == "blockwise":
        # weight scales are per 128 x 128 tile: dequantize whole 128-row bands that contain the sampled columns
        bands = np.unique(cols // 128)
        w_rows = np.concatenate([np.arange(b * 128, (b + 1) * 128) for b in bands])
        w_band = oq.dequantize_fp8_blockwise_weight(u8(qw[w_rows]), f32(sw[bands]), "e4m3")
        pos = {int(r): i for i, r in enumerate(w_rows)}
        ref = og.gemm_nt(a_deq(rows), w_band[[pos[int(cc)] for cc in cols]])
    else:
        ref = og.gemm_nt(a_deq(rows), w_deq(cols))
    got = f32(c[rows][:, cols])
    assert og.rel_frobenius(got, ref) <= 1e-2
    # the reference's accuracy gate against the unquantized product
    assert og.snr_db(got, f32(a[rows]) @ f32(w[cols]).T) > 25
    # determinism
    assert torch.equal(c, run(qa, sa))
    # permuting the rows of A permutes the rows of C, bit for bit (each output element sums K in the same order)
    perm = torch.randperm(M, generator=torch.Generator().manual_seed(8)).cuda()
    if gran == "tensorwise":
        cp = run(qa[perm].contiguous(), sa)
    elif gran == "blockwise":
        cp = run(qa[perm].contiguous(), sa[perm].contiguous())
    else:
        cp = run(qa[perm].contiguous(), sa[perm].contiguous())
    nv.check_status(c.device)
    assert torch.equal(cp, c[perm])


def test_mxfp4_gemm_sampled_outputs(mods, operands):
    """MXFP4 forward at the benchmark shape: sampled outputs against the dequantized operands (tolerance 5e-2 stated for
    FP4; the products themselves are exact, so the bf16 rounding of the output dominates)."""
    qi, _, nv, _, SR = mods
    from primus_turbo.pytorch.kernels.gemm.gemm_fp4_impl import gemm_fp4_impl
    a, w = operands
    fp4 = torch.float4_e2m1fn_x2
    qa, sa = qi.quantize_mxfp4_impl(a, fp4, 1, 32)
    qw, sw = qi.quantize_mxfp4_impl(w, fp4, 1, 32)
    c = gemm_fp4_impl(qa, sa, False, qw, sw, True, torch.bfloat16, False)
    nv.check_status(c.device)
    rows, cols = _rows(M, 64, 11), _rows(N, 64, 12)
    qa8, qw8 = qa.view(torch.uint8), qw.view(torch.uint8)  # torch cannot index packed-fp4 tensors
    ref = og.gemm_nt(oq.dequantize_mx(u8(qa8[rows]), u8(sa[rows]), "e2m1"), oq.dequantize_mx(u8(qw8[cols]), u8(sw[cols]), "e2m1"))
    assert og.rel_frobenius(f32(c[rows][:, cols]), ref) <= 1e-2
    assert torch.equal(c, gemm_fp4_impl(qa, sa, False, qw, sw, True, torch.bfloat16, False))


def test_tensorwise_gemm_is_linear_in_the_scale(mods, operands):
    qi, gi, nv, SG, _ = mods
    a, w = operands
    (qa, sa), (qw, sw) = qi.quantize_fp8_tensorwise_impl(a, F8), qi.quantize_fp8_tensorwise_impl(w, F8)
    c1 = gi.gemm_fp8_impl(qa, sa, False, qw, sw, True, torch.bfloat16, False, SG.TENSORWISE)
    c4 = gi.gemm_fp8_impl(qa, sa * 4, False, qw, sw, True, torch.bfloat16, False, SG.TENSORWISE)
    nv.check_status(c1.device)
    assert torch.equal(c4, c1 * 4)  # a power of two only shifts the exponent of every output


def test_grouped_blockwise_moe_shape_sampled(mods):
    """MoE grouped forward at the shape of the grouped benchmark config: 8 experts, 64k tokens, 2048 -> 1408."""
    qi, gi, nv, SG, _ = mods
    from primus_turbo.pytorch.kernels.grouped_gemm import grouped_gemm_fp8_impl as ggi
    G, tokens, Kd, Nd = 8, 65536, 2048, 1408
    lens = torch.tensor([9000, 7384, 8192, 8192, 10000, 6384, 8192, 8192], dtype=torch.int64)
    assert int(lens.sum()) == tokens
    a = make((tokens, Kd), torch.bfloat16, 103, "outlier")
    w = make((G, Nd, Kd), torch.bfloat16, 104, "weight")
    lens_d = lens.cuda()
    offs = torch.zeros(G + 1, dtype=torch.int64)
    offs[1:] = torch.cumsum(lens, 0)
    offs_d = offs.cuda()
    qa, sa = qi.quant_fp8_blockwise_impl(a, F8, 1)
    qw, sw = qi.quant_fp8_blockwise_for_weight_impl(w, F8)
    c = ggi.grouped_gemm_fp8_impl(qa, qw, sa, sw, lens_d, offs_d, False, True, torch.bfloat16, SG.BLOCKWISE)
    nv.check_status(c.device)
    rng = np.random.default_rng(9)
    for g in (0, 3, 7):
        lo, hi = int(offs[g]), int(offs[g + 1])
        rows = np.sort(rng.choice(np.arange(lo, hi), size=32, replace=False))
        a_deq = oq.dequantize_fp8_blockwise(u8(qa[rows]), f32(sa[rows]), "e4m3", 1)
        w_deq = oq.dequantize_fp8_blockwise_weight(u8(qw[g]), f32(sw[g]), "e4m3")
        ref = og.gemm_nt(a_deq, w_deq)
        assert og.rel_frobenius(f32(c[rows]), ref) <= 1e-2, f"group {g}"
