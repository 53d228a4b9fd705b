"""Pre-shuffled MX layouts: the numpy restatement against hand-computed positions (CPU), and the CUDA kernels and the
quantizers' shuffle options against the restatement (B200), bit for bit."""
import numpy as np
import pytest
import torch

from oracle import layout_shuffle as O


def test_scale_positions_by_hand():
    s = (np.arange(40 * 10) % 251).astype(np.uint8).reshape(40, 10)
    o = O.shuffle_scale(s)
    assert o.shape == (256, 16)
    f = o.ravel()
    # index = i0 * (N_pad / 8) * 256 + i3 * 256 + i5 * 64 + i2 * 4 + i4 * 2 + i1
    assert f[0] == s[0, 0] and f[1] == s[16, 0] and f[2] == s[0, 4] and f[3] == s[16, 4]
    assert f[4] == s[1, 0] and f[64] == s[0, 1] and f[256] == s[0, 8] and f[512] == s[32, 0]
    assert f[256 + 3 * 64 + 15 * 4 + 3] == 0          # (row 31, col 15): column padding
    assert int(np.count_nonzero(o)) == int(np.count_nonzero(s))


def test_codes_positions_by_hand():
    c = (np.arange(32 * 64) % 253).astype(np.uint8).reshape(32, 64)
    f = O.shuffle_codes(c).ravel()
    # index = (row / 16) * (K * 16) + (col / 32) * 512 + ((col % 32) / 16) * 256 + (row % 16) * 16 + col % 16
    assert f[0] == c[0, 0] and f[15] == c[0, 15] and f[16] == c[1, 0] and f[256] == c[0, 16]
    assert f[512] == c[0, 32] and f[1024] == c[16, 0] and f[1024 + 512 + 256 + 15 * 16 + 15] == c[31, 63]
    assert sorted(f.tolist()) == sorted(c.ravel().tolist())


def _ops():
    import primus_turbo.pytorch as turbo
    return turbo.ops


@pytest.mark.gpu
@pytest.mark.parametrize("M,N", [(32, 1), (64, 8), (100, 9), (256, 32), (1000, 37), (4096, 224)])
def test_shuffle_scale_matches_oracle(M, N):
    g = torch.Generator().manual_seed(M * 131 + N)
    s = torch.randint(0, 256, (M, N), dtype=torch.uint8, generator=g)
    out = _ops().shuffle_scale(s.cuda().view(torch.float8_e8m0fnu))
    assert out.dtype == torch.float8_e8m0fnu
    assert np.array_equal(out.view(torch.uint8).cpu().numpy(), O.shuffle_scale(s.numpy()))


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float4_e2m1fn_x2, torch.float8_e4m3fn])
@pytest.mark.parametrize("M,K", [(16, 32), (32, 64), (256, 512), (1024, 2048)])
def test_shuffle_weight_matches_oracle(dtype, M, K):
    g = torch.Generator().manual_seed(M * 7 + K)
    c = torch.randint(0, 256, (M, K), dtype=torch.uint8, generator=g)
    out = _ops().shuffle_weight(c.cuda().view(dtype))
    assert out.dtype == dtype and out.shape == (M, K)
    assert np.array_equal(out.view(torch.uint8).cpu().numpy(), O.shuffle_codes(c.numpy()))
    with pytest.raises(AssertionError):
        _ops().shuffle_weight(c[:M - 1].contiguous().cuda().view(dtype))


@pytest.mark.gpu
@pytest.mark.parametrize("fp4", [False, True])
@pytest.mark.parametrize("M,N", [(32, 64), (256, 256), (1024, 1024), (96, 160)])
@pytest.mark.parametrize("two_d", [False, True])
def test_quantizer_shuffle_options_equal_shuffling_the_plain_outputs(fp4, M, N, two_d):
    """The reference's own check (tests/pytorch/ops/test_quantization.py:500-560): quantize with shuffle_scale, and
    shuffle_scale of the plain scales, give the same bytes; here also for the codes (shuffle_out)."""
    from primus_turbo.pytorch.core.low_precision import ScalingGranularity, ScalingRecipe
    ops = _ops()
    x = torch.randn(M, N, device="cuda", dtype=torch.bfloat16, generator=torch.Generator(device="cuda").manual_seed(42))
    q = ops.quantize_fp4_with_trans if fp4 else ops.quantize_fp8_with_trans
    dt = torch.float4_e2m1fn_x2 if fp4 else torch.float8_e4m3fn
    plain_r = ScalingRecipe(use_2d_block=two_d)
    shuf_r = ScalingRecipe(use_2d_block=two_d, shuffle_scale=True, shuffle_out=True)
    kw = dict(granularity=ScalingGranularity.MX_BLOCKWISE, block_size=32)
    qr, sr, qc, sc = q(x, dt, scaling_recipe=plain_r, scaling_recipe_for_trans=plain_r, **kw)
    qr2, sr2, qc2, sc2 = q(x, dt, scaling_recipe=shuf_r, scaling_recipe_for_trans=shuf_r, **kw)
    u8 = lambda t: t.view(torch.uint8)
    assert torch.equal(u8(ops.shuffle_scale(sr)), u8(sr2)) and torch.equal(u8(ops.shuffle_scale(sc)), u8(sc2))
    assert torch.equal(u8(ops.shuffle_weight(qr)), u8(qr2)) and torch.equal(u8(ops.shuffle_weight(qc)), u8(qc2))
    assert np.array_equal(u8(sr2).cpu().numpy(), O.shuffle_scale(u8(sr).cpu().numpy()))
    assert np.array_equal(u8(qc2).cpu().numpy(), O.shuffle_codes(u8(qc).cpu().numpy()))
