"""Parity at the shapes of the three large benchmark configurations, where the oracle cannot restate the whole
problem: C3 (MXFP8 16384 x 28672 x 8192, forward + wgrad from the transposed copies), C4 (blockwise-FP8 MoE, 256
experts, 131072 rows, Zipf group lengths with empty groups, gate_up 7168 -> 4096 and down 2048 -> 7168) and C5 (MXFP4
MoE, 8 experts, 65536 rows, Dirichlet group lengths, 4096 -> 14336).

Operands are drawn on the device (seeded); the compared rows, columns and 128-row bands are downloaded, so oracle and
kernels see identical bits.  Quantizers are checked bit for bit on the sampled pieces (a 1-D block depends on its
row / column band only), GEMM outputs against the fp32 product of the dequantized operands at the sampled positions:
relative Frobenius error <= 1e-2 for FP8, <= 5e-2 for FP4.
"""
import numpy as np
import pytest
import torch

import bench_configs as bc
from oracle import gemm as og
from oracle import quant as oq
from tests._util import assert_bits_equal, f32, u8

pytestmark = pytest.mark.gpu

F8, F5, F4 = torch.float8_e4m3fn, torch.float8_e5m2, torch.float4_e2m1fn_x2
DEV = "cuda"


@pytest.fixture(scope="module")
def mods():
    from primus_turbo.pytorch.core.low_precision import ScalingGranularity, ScalingRecipe
    from primus_turbo.pytorch.kernels import _native as nv
    from primus_turbo.pytorch.kernels.gemm import gemm_fp8_impl as gi
    from primus_turbo.pytorch.kernels.grouped_gemm import grouped_gemm_fp4_impl as gg4
    from primus_turbo.pytorch.kernels.grouped_gemm import grouped_gemm_fp8_impl as ggi
    from primus_turbo.pytorch.kernels.quantization import quantization_impl as qi
    return dict(qi=qi, gi=gi, ggi=ggi, gg4=gg4, nv=nv, SG=ScalingGranularity, SR=ScalingRecipe)


def _pick(n, count, seed):
    return np.sort(np.random.default_rng(seed).choice(n, size=min(count, n), replace=False))


def _idx(a):
    return torch.as_tensor(np.asarray(a), dtype=torch.int64, device=DEV)


# ------------------------------------------------------------------------------------------------ generators
def test_group_length_generators():
    lens = bc.zipf_group_lens()
    assert lens.shape == (256,) and lens.sum() == 131072 and (lens == 0).sum() >= 4
    assert lens.max() > 4 * lens[lens > 0].mean()          # Zipf skew: the busiest expert is far above the mean
    assert np.array_equal(lens, bc.zipf_group_lens())      # seeded
    l5 = bc.dirichlet_group_lens()
    assert l5.shape == (8,) and l5.sum() == 65536 and l5.min() >= 0


# ------------------------------------------------------------------------------------------------ C3
def test_c3_mxfp8_forward_and_wgrad(mods):
    qi, gi, nv, SG, SR = mods["qi"], mods["gi"], mods["nv"], mods["SG"], mods["SR"]
    M, K, N = bc.C3["M"], bc.C3["K"], bc.C3["N"]
    x = bc.randn_bf16((M, K), 1.0, 71, DEV)
    w = bc.randn_bf16((N, K), 0.01, 72, DEV)
    two_d = SR(use_2d_block=True)
    a_row, a_row_s, a_col, a_col_s = qi.quantize_mxfp8_impl(x, F8, None, 32, True)
    b_row, b_row_s, _, _ = qi.quantize_mxfp8_impl(w, F8, None, 32, True, two_d, two_d)
    # quantizer, bit exact on sampled rows (row copy) and sampled columns (transposed copy)
    rows = _pick(M, 24, 1)
    wq, ws = oq.quantize_mx(f32(x[_idx(rows)]), "e4m3", 1)
    assert_bits_equal(u8(a_row[_idx(rows)]), wq, "C3 row bytes")
    assert_bits_equal(u8(a_row_s[_idx(rows)]), ws, "C3 row scales")
    cols = _pick(K, 32, 2)
    wq, ws = oq.quantize_mx(f32(x[:, _idx(cols)]), "e4m3", 0)
    assert_bits_equal(u8(a_col[_idx(cols)]), wq, "C3 transposed bytes")
    assert_bits_equal(u8(a_col_s[_idx(cols)]), ws, "C3 transposed scales")
    # 2-D weight scales: whole 32-row bands
    band = int(_pick(N // 32, 1, 3)[0]) * 32
    wq, ws = oq.quantize_mx(f32(w[band:band + 32]), "e4m3", 1, True)
    assert_bits_equal(u8(b_row[band:band + 32]), wq, "C3 weight bytes (2-D scales)")
    assert_bits_equal(u8(b_row_s[band:band + 32]), ws, "C3 weight scales (2-D)")
    # forward
    c = gi.gemm_fp8_impl(a_row, a_row_s, False, b_row, b_row_s, True, torch.bfloat16, False, SG.MX_BLOCKWISE)
    nv.check_status(c.device)
    r, cc = _pick(M, 48, 4), _pick(N, 48, 5)
    ref = og.gemm_nt(oq.dequantize_mx(u8(a_row[_idx(r)]), u8(a_row_s[_idx(r)]), "e4m3"),
                     oq.dequantize_mx(u8(b_row[_idx(cc)]), u8(b_row_s[_idx(cc)]), "e4m3"))
    assert og.rel_frobenius(f32(c[_idx(r)][:, _idx(cc)]), ref) <= 1e-2
    del c, b_row, w
    # wgrad: dW [N, K] = dY_col [N, M] . X_col [K, M]^T with e5m2 gradients (HYBRID)
    dy = bc.randn_bf16((M, N), 1e-3, 73, DEV)
    _, _, g_col, g_col_s = qi.quantize_mxfp8_impl(dy, F5, None, 32, True)
    cols_n = _pick(N, 32, 6)
    wq, ws = oq.quantize_mx(f32(dy[:, _idx(cols_n)]), "e5m2", 0)
    assert_bits_equal(u8(g_col[_idx(cols_n)]), wq, "C3 gradient transposed bytes")
    assert_bits_equal(u8(g_col_s[_idx(cols_n)]), ws, "C3 gradient transposed scales")
    del dy
    dw = gi.gemm_fp8_impl(g_col, g_col_s, False, a_col, a_col_s, True, torch.bfloat16, False, SG.MX_BLOCKWISE)
    nv.check_status(dw.device)
    rn, ck = _pick(N, 40, 7), _pick(K, 40, 8)
    ref = og.gemm_nt(oq.dequantize_mx(u8(g_col[_idx(rn)]), u8(g_col_s[_idx(rn)]), "e5m2"),
                     oq.dequantize_mx(u8(a_col[_idx(ck)]), u8(a_col_s[_idx(ck)]), "e4m3"))
    assert og.rel_frobenius(f32(dw[_idx(rn)][:, _idx(ck)]), ref) <= 1e-2


# ------------------------------------------------------------------------------------------------ C4
@pytest.mark.parametrize("projection", ["gate_up", "down"])
def test_c4_blockwise_grouped_fwd_dgrad_wgrad(mods, projection):
    qi, ggi, nv, SG = mods["qi"], mods["ggi"], mods["nv"], mods["SG"]
    G, rows = bc.C4["G"], bc.C4["rows"]
    N, K = (bc.C4["inter2"], bc.C4["hidden"]) if projection == "gate_up" else (bc.C4["hidden"], bc.C4["inter"])
    lens = bc.zipf_group_lens()
    offs_h = np.concatenate([[0], np.cumsum(lens)])
    lens_t, offs = bc.offsets_of(lens, DEV)
    x = bc.randn_bf16((rows, K), 1.0, 81, DEV)
    w = bc.randn_bf16((G, N, K), 0.02, 83, DEV)
    a_row, a_col, a_s_row, a_s_col, plens, poffs = qi.quant_fp8_blockwise_segment_m_row_col_impl(x, F8, 128, lens_t, offs)
    poffs_h = poffs.cpu().numpy()
    assert np.array_equal(poffs_h, np.concatenate([[0], np.cumsum((lens + 127) // 128 * 128)])), "padded offsets"
    # groups under test: the largest, one empty, the last non-empty, two random ones
    nonempty = np.flatnonzero(lens > 0)
    small = [int(g) for g in nonempty if lens[g] <= 384]
    groups = sorted({int(np.argmax(lens)), int(np.flatnonzero(lens == 0)[0]), int(nonempty[-1]), small[0], small[-1],
                     *[int(g) for g in np.random.default_rng(9).choice(nonempty, 2, replace=False)]})
    w_q, w_s = qi.quant_fp8_blockwise_for_weight_impl(w, F8)
    # ---- segment-M quantizer, bit exact: row copy rows of the group; column copy = the group's 128-padded segment
    for g in groups:
        lo, hi, n = int(offs_h[g]), int(offs_h[g + 1]), int(lens[g])
        if n == 0:
            assert poffs_h[g] == poffs_h[g + 1]
            continue
        take = np.arange(lo, min(hi, lo + 192))           # first rows of the group: a whole band and a ragged one
        wq, ws = oq.quantize_fp8_blockwise(f32(x[take[0]:take[-1] + 1]), "e4m3", 1)
        assert_bits_equal(u8(a_row[take[0]:take[-1] + 1]), wq, f"C4 row bytes, group {g}")
        assert_bits_equal(f32(a_s_row[:, take[0]:take[-1] + 1]).T.copy(), ws, f"C4 row scales (transposed layout), group {g}")
        # last (ragged) 128-row band of the group's column copy: rows past the group's end are zeros
        last = (n - 1) // 128 * 128
        seg = np.zeros((128, K), dtype=np.float32)
        seg[: n - last] = f32(x[lo + last:hi])
        wq, ws = oq.quantize_fp8_blockwise(seg, "e4m3", 0)
        p0 = int(poffs_h[g]) + last
        assert_bits_equal(u8(a_col[p0:p0 + 128]), wq, f"C4 column bytes, last band of group {g}")
        assert_bits_equal(f32(a_s_col[p0 // 128:p0 // 128 + 1]), ws, f"C4 column scales, last band of group {g}")
    # ---- forward
    out = ggi.grouped_gemm_fp8_impl(a_row, w_q, a_s_row, w_s, lens_t, offs, False, True, torch.bfloat16, SG.BLOCKWISE)
    nv.check_status(out.device)
    rng = np.random.default_rng(10)
    for g in groups:
        lo, hi = int(offs_h[g]), int(offs_h[g + 1])
        if hi == lo:
            continue
        r = np.sort(rng.choice(np.arange(lo, hi), size=min(24, hi - lo), replace=False))
        a_deq = oq.dequantize_fp8_blockwise(u8(a_row[_idx(r)]), f32(a_s_row[:, _idx(r)]).T.copy(), "e4m3", 1)
        nb = int(rng.integers(N // 128))      # one 128-wide band of output columns: whole weight tiles
        w_deq = oq.dequantize_fp8_blockwise_weight(u8(w_q[g][nb * 128:(nb + 1) * 128]), f32(w_s[g][nb:nb + 1]), "e4m3")
        got = f32(out[_idx(r)][:, nb * 128:(nb + 1) * 128])
        assert og.rel_frobenius(got, og.gemm_nt(a_deq, w_deq)) <= 1e-2, f"C4 forward, group {g}"
    del out, x
    # ---- dgrad: dX = dY . W  (weight read MN-major in place), e5m2 gradients
    dy = bc.randn_bf16((rows, N), 1e-3, 82, DEV)
    g_row, g_col, g_s_row, g_s_col, _, _ = qi.quant_fp8_blockwise_segment_m_row_col_impl(dy, F5, 128, lens_t, offs)
    del dy
    dx = ggi.grouped_gemm_fp8_impl(g_row, w_q, g_s_row, w_s, lens_t, offs, False, False, torch.bfloat16, SG.BLOCKWISE)
    nv.check_status(dx.device)
    for g in groups:
        lo, hi = int(offs_h[g]), int(offs_h[g + 1])
        if hi == lo:
            continue
        r = np.sort(rng.choice(np.arange(lo, hi), size=min(16, hi - lo), replace=False))
        g_deq = oq.dequantize_fp8_blockwise(u8(g_row[_idx(r)]), f32(g_s_row[:, _idx(r)]).T.copy(), "e5m2", 1)
        kb = int(rng.integers(K // 128))      # one 128-wide band of input features: whole weight tiles
        w_deq = oq.dequantize_fp8_blockwise_weight(u8(w_q[g][:, kb * 128:(kb + 1) * 128]), f32(w_s[g][:, kb:kb + 1]), "e4m3")
        assert og.rel_frobenius(f32(dx[_idx(r)][:, kb * 128:(kb + 1) * 128]), g_deq @ w_deq) <= 1e-2, f"C4 dgrad, group {g}"
    del dx, g_row
    # ---- wgrad (variable K): dW[g] = dY_g^T . X_g over the group's padded segment -> [N, K]; empty group -> zeros
    dw = ggi.grouped_gemm_fp8_variable_k_impl(a_col, g_col, a_s_col, g_s_col, plens, poffs, True, False, True, torch.bfloat16,
                                              SG.BLOCKWISE)
    nv.check_status(dw.device)
    for g in groups:
        p0, p1 = int(poffs_h[g]), int(poffs_h[g + 1])
        if p1 == p0:
            assert int(torch.count_nonzero(dw[g])) == 0, f"C4 wgrad of empty group {g} is not zero"
            continue
        # the whole contraction (every padded row of the group) for sampled output rows / columns: column scales are
        # per column, so the sampled columns are dequantized alone
        rn, ck = _pick(N, 64, 11 + g), _pick(K, 64, 12 + g)
        a_deq = oq.dequantize_fp8_blockwise(u8(a_col[p0:p1][:, _idx(ck)]), f32(a_s_col[p0 // 128:p1 // 128][:, _idx(ck)]), "e4m3", 0)
        g_deq = oq.dequantize_fp8_blockwise(u8(g_col[p0:p1][:, _idx(rn)]), f32(g_s_col[p0 // 128:p1 // 128][:, _idx(rn)]), "e5m2", 0)
        ref = g_deq.T @ a_deq
        assert og.rel_frobenius(f32(dw[g][_idx(rn)][:, _idx(ck)]), ref) <= 1e-2, f"C4 wgrad, group {g}"


def test_c4_grouped_mx_quantize_at_256_groups(mods):
    """The grouped MX quantizer keeps its offset tables in shared memory for up to 256 groups: C4's group count sits
    exactly on that limit.  Sampled groups (one empty, the last) against the oracle, bit exact."""
    qi = mods["qi"]
    G, K = bc.C4["G"], 512
    lens = bc.zipf_group_lens(G, 32768, seed=bc.C4["seed"])
    lens_t, offs = bc.offsets_of(lens, DEV)
    offs_h = np.concatenate([[0], np.cumsum(lens)])
    x = bc.randn_bf16((32768, K), 1.0, 85, DEV)
    q_row, s_row, q_col, s_col, _, orow, _, ocol = qi.grouped_quantize_mxfp8_impl(x, F8, None, 32, lens_t, offs, with_trans=True)
    orow_h, ocol_h = orow.cpu().numpy(), ocol.cpu().numpy()
    nonempty = np.flatnonzero(lens > 0)
    for g in (int(nonempty[0]), int(nonempty[len(nonempty) // 2]), int(nonempty[-1]), int(np.argmax(lens))):
        lo, hi, n = int(offs_h[g]), int(offs_h[g + 1]), int(lens[g])
        wq, ws, _, _ = oq.quantize_mx_grouped(f32(x[lo:hi]), "e4m3", [n], 1)
        assert_bits_equal(u8(q_row[orow_h[g]:orow_h[g] + n]), wq[:n], f"grouped MX row bytes, group {g}")
        assert_bits_equal(u8(s_row[orow_h[g]:orow_h[g] + n]), ws[:n], f"grouped MX row scales, group {g}")
        wq, ws, _, _ = oq.quantize_mx_grouped(f32(x[lo:hi]), "e4m3", [n], 0)
        c0, c1 = int(ocol_h[g]), int(ocol_h[g + 1])
        assert_bits_equal(u8(q_col[:, c0:c1]), wq, f"grouped MX column bytes, group {g}")
        assert_bits_equal(u8(s_col[:, c0 // 32:c1 // 32]), ws, f"grouped MX column scales, group {g}")


# ------------------------------------------------------------------------------------------------ C5
def test_c5_mxfp4_grouped_fwd_dgrad_wgrad(mods):
    qi, gg4, nv, SR = mods["qi"], mods["gg4"], mods["nv"], mods["SR"]
    G, rows, K, N = bc.C5["G"], bc.C5["rows"], bc.C5["hidden"], bc.C5["ffn"]
    lens = bc.dirichlet_group_lens()
    offs_h = np.concatenate([[0], np.cumsum(lens)])
    lens_t, offs = bc.offsets_of(lens, DEV)
    x = bc.randn_bf16((rows, K), 1.0, 91, DEV)
    w = bc.randn_bf16((G, N, K), 0.02, 93, DEV)
    rht, two_d = SR(use_rht=True), SR(use_2d_block=True)
    a_row, a_s_row, a_col, a_s_col, _, orow, lcol, ocol = qi.grouped_quantize_mxfp4_impl(
        x, F4, None, 32, lens_t, offs, with_trans=True, scaling_recipe=SR(), scaling_recipe_for_trans=rht)
    w_row, w_s_row, w_col, w_s_col = qi.quantize_mxfp4_impl(w, F4, None, 32, with_trans=True, scaling_recipe=two_d,
                                                            scaling_recipe_for_trans=two_d)
    a8, w8 = a_row.view(torch.uint8), w_row.view(torch.uint8)
    ocol_h = ocol.cpu().numpy()
    nonempty = [int(g) for g in np.flatnonzero(lens > 0)]
    groups = sorted({nonempty[0], nonempty[-1], int(np.argmax(lens)), int(np.argmin(np.where(lens > 0, lens, 1 << 40)))})
    # quantizer, bit exact: tight row copy on sampled rows; transposed + Hadamard copy on the smallest group
    r = _pick(rows, 32, 21)
    wq, ws = oq.quantize_mx(f32(x[_idx(r)]), "e2m1", 1)
    assert_bits_equal(u8(a8[_idx(r)]), wq, "C5 row bytes")
    assert_bits_equal(u8(a_s_row[_idx(r)]), ws, "C5 row scales")
    gs = groups[0] if lens[groups[0]] <= 4096 else int(np.argmin(np.where(lens > 0, lens, 1 << 40)))
    lo, hi, n = int(offs_h[gs]), int(offs_h[gs + 1]), int(lens[gs])
    if 0 < n <= 8192:
        wq, ws, _, _ = oq.quantize_mx_grouped(f32(x[lo:hi]), "e2m1", [n], 0, use_rht=True, col_align=256)
        c0, c1 = int(ocol_h[gs]), int(ocol_h[gs + 1])
        assert_bits_equal(u8(a_col.view(torch.uint8)[:, c0 // 2:c1 // 2]), wq, f"C5 transposed bytes (RHT), group {gs}")
        assert_bits_equal(u8(a_s_col[:, c0 // 32:c1 // 32]), ws, f"C5 transposed scales (RHT), group {gs}")
    # forward
    out = gg4.grouped_gemm_fp4_impl(a_row, w_row, a_s_row, w_s_row, lens_t, orow, out_dtype=torch.bfloat16, group_offs_out=offs)
    nv.check_status(out.device)
    rng = np.random.default_rng(22)
    for g in groups:
        lo, hi = int(offs_h[g]), int(offs_h[g + 1])
        rr = np.sort(rng.choice(np.arange(lo, hi), size=min(24, hi - lo), replace=False))
        cc = _pick(N, 48, 23 + g)
        ref = og.gemm_nt(oq.dequantize_mx(u8(a8[_idx(rr)]), u8(a_s_row[_idx(rr)]), "e2m1"),
                         oq.dequantize_mx(u8(w8[g][_idx(cc)]), u8(w_s_row[g][_idx(cc)]), "e2m1"))
        assert og.rel_frobenius(f32(out[_idx(rr)][:, _idx(cc)]), ref) <= 5e-2, f"C5 forward, group {g}"
    del out
    # dgrad: dX = dY . W through the transposed weight copy [G, K, N/2]
    dy = bc.randn_bf16((rows, N), 1.0, 92, DEV)
    g_row, g_s_row, g_col, g_s_col, _, orow2, _, _ = qi.grouped_quantize_mxfp4_impl(
        dy, F4, None, 32, lens_t, offs, with_trans=True, scaling_recipe=SR(), scaling_recipe_for_trans=rht)
    del dy
    dx = gg4.grouped_gemm_fp4_impl(g_row, w_col, g_s_row, w_s_col, lens_t, orow2, out_dtype=torch.bfloat16, group_offs_out=offs)
    nv.check_status(dx.device)
    g8, wc8 = g_row.view(torch.uint8), w_col.view(torch.uint8)
    for g in groups:
        lo, hi = int(offs_h[g]), int(offs_h[g + 1])
        rr = np.sort(rng.choice(np.arange(lo, hi), size=min(16, hi - lo), replace=False))
        ck = _pick(K, 48, 24 + g)
        ref = og.gemm_nt(oq.dequantize_mx(u8(g8[_idx(rr)]), u8(g_s_row[_idx(rr)]), "e2m1"),
                         oq.dequantize_mx(u8(wc8[g][_idx(ck)]), u8(w_s_col[g][_idx(ck)]), "e2m1"))
        assert og.rel_frobenius(f32(dx[_idx(rr)][:, _idx(ck)]), ref) <= 5e-2, f"C5 dgrad, group {g}"
    del dx
    # wgrad (variable K over 256-padded token segments, both operands Hadamard-transformed along the tokens)
    dw = gg4.grouped_gemm_fp4_variable_k_impl(g_col, a_col, g_s_col, a_s_col, lcol, ocol, torch.bfloat16)
    nv.check_status(dw.device)
    gc8, ac8 = g_col.view(torch.uint8), a_col.view(torch.uint8)
    for g in groups:
        c0, c1 = int(ocol_h[g]), int(ocol_h[g + 1])
        rn, ck = _pick(N, 32, 25 + g), _pick(K, 32, 26 + g)
        ref = og.gemm_nt(oq.dequantize_mx(u8(gc8[_idx(rn)][:, c0 // 2:c1 // 2]), u8(g_s_col[_idx(rn)][:, c0 // 32:c1 // 32]), "e2m1"),
                         oq.dequantize_mx(u8(ac8[_idx(ck)][:, c0 // 2:c1 // 2]), u8(a_s_col[_idx(ck)][:, c0 // 32:c1 // 32]), "e2m1"))
        assert og.rel_frobenius(f32(dw[g][_idx(rn)][:, _idx(ck)]), ref) <= 5e-2, f"C5 wgrad, group {g}"
