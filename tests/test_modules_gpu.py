"""Float8Linear and the grouped low-precision linear layers: same results as calling the operators directly, gradients
against an fp32 reference, and the quantized-weight cache (reuse between optimizer steps, gradient still reaches the
parameter).  Module surface: primus_turbo/pytorch/modules/linear_fp8.py and grouped_linear.py of the reference."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def snr(x, ref):
    x, ref = x.detach().float(), ref.detach().float()
    return float(10 * torch.log10(ref.pow(2).sum() / (x - ref).pow(2).sum().clamp_min(1e-30)))


@pytest.fixture(scope="module")
def m():
    import primus_turbo.pytorch as turbo
    from primus_turbo.pytorch.core.low_precision import (Float4QuantConfig, Float8QuantConfig, Format, ScaleDtype,
                                                         ScalingGranularity)
    from primus_turbo.pytorch.modules import _weight_cache
    return dict(turbo=turbo, Cfg=Float8QuantConfig, Cfg4=Float4QuantConfig, Format=Format, SD=ScaleDtype,
                SG=ScalingGranularity, wc=_weight_cache)


def _cfg(m, gran):
    kw = {}
    if gran == "BLOCKWISE":
        kw["block_size"] = 128
    if gran == "MX_BLOCKWISE":
        kw.update(block_size=32, scale_dtype=m["SD"].E8M0)
    return m["Cfg"](format=m["Format"].E4M3, granularity=m["SG"][gran], **kw)


GRANS = ["TENSORWISE", "ROWWISE", "BLOCKWISE", "MX_BLOCKWISE"]


@pytest.mark.parametrize("gran", GRANS)
@pytest.mark.parametrize("bias", [True, False])
def test_float8_linear_matches_op_and_reference(m, gran, bias):
    turbo = m["turbo"]
    torch.manual_seed(1)
    cfg = _cfg(m, gran)
    lin = turbo.modules.Float8Linear(256, 384, bias=bias, config=cfg, device="cuda", dtype=torch.bfloat16)
    x = torch.randn(4, 96, 256, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    y = lin(x)
    assert y.shape == (4, 96, 384)
    direct = turbo.ops.gemm_fp8(x.detach().reshape(-1, 256), lin.weight.detach(), trans_b=True, out_dtype=torch.bfloat16, config=cfg)
    if bias:
        direct = direct + lin.bias
    assert torch.equal(y.detach().reshape(-1, 384), direct)
    ref = torch.nn.Linear(256, 384, bias=bias, device="cuda", dtype=torch.bfloat16)
    with torch.no_grad():
        ref.weight.copy_(lin.weight)
        if bias:
            ref.bias.copy_(lin.bias)
    x_ref = x.detach().clone().requires_grad_()
    y_ref = ref(x_ref)
    go = torch.randn_like(y)
    y.backward(go)
    y_ref.backward(go)
    assert snr(y, y_ref) > 25 and snr(x.grad, x_ref.grad) > 25 and snr(lin.weight.grad, ref.weight.grad) > 25
    if bias:
        assert snr(lin.bias.grad, ref.bias.grad) > 40


def test_float8_linear_from_float(m):
    turbo = m["turbo"]
    cfg = _cfg(m, "BLOCKWISE")
    base = torch.nn.Linear(128, 256, device="cuda", dtype=torch.bfloat16)
    copy = turbo.modules.Float8Linear.from_float(base, cfg, inplace=False)
    assert type(base) is torch.nn.Linear and isinstance(copy, turbo.modules.Float8Linear)
    assert torch.equal(copy.weight, base.weight) and copy.weight is not base.weight
    same = turbo.modules.Float8Linear.from_float(base, cfg)
    assert same is base and isinstance(base, turbo.modules.Float8Linear) and base.config is cfg
    x = torch.randn(64, 128, device="cuda", dtype=torch.bfloat16)
    assert torch.equal(base(x), copy(x))
    assert "config=" in repr(base)


@pytest.mark.parametrize("gran", GRANS)
def test_float8_linear_weight_cache(m, gran, monkeypatch):
    turbo, wc = m["turbo"], m["wc"]
    torch.manual_seed(2)
    cfg = _cfg(m, gran)
    plain = turbo.modules.Float8Linear(256, 384, bias=False, config=cfg, device="cuda", dtype=torch.bfloat16)
    cached = turbo.modules.Float8Linear.from_float(plain, cfg, inplace=False, cache_quantized_weight=True)
    calls = []
    real = wc.create_quantized_weight
    monkeypatch.setattr(wc, "create_quantized_weight", lambda *a, **k: (calls.append(1), real(*a, **k))[1])
    x = torch.randn(192, 256, device="cuda", dtype=torch.bfloat16)
    go = torch.randn(192, 384, device="cuda", dtype=torch.bfloat16)
    for step in range(3):   # three micro-batches, one quantization
        xa, xb = x.clone().requires_grad_(), x.clone().requires_grad_()
        ya, yb = plain(xa), cached(xb)
        assert torch.equal(ya, yb)
        ya.backward(go)
        yb.backward(go)
        assert snr(xb.grad, xa.grad) > 30
    assert len(calls) == 1
    assert cached.weight.grad is not None and snr(cached.weight.grad, plain.weight.grad) > 30
    with torch.no_grad():   # an optimizer step writes in place: the cache must notice
        cached.weight.add_(0.5)
        plain.weight.add_(0.5)
    assert torch.equal(plain(x), cached(x))
    assert len(calls) == 2
    with torch.no_grad():   # inference: forward copy only
        assert torch.equal(plain(x), cached(x))
        # a write around the version counter is invisible to the cache until it is cleared
        cached.weight.data.mul_(2.0)
        plain.weight.data.mul_(2.0)
        cached.clear_quantized_weight_cache()
        assert torch.equal(plain(x), cached(x))


@pytest.mark.parametrize("gran", GRANS + ["FP4"])
@pytest.mark.parametrize("cache", [False, True])
def test_grouped_linear_modules(m, gran, cache):
    turbo = m["turbo"]
    torch.manual_seed(3)
    lens = [160, 0, 96, 256]
    G, M, K, N = len(lens), sum(lens), 256, 384
    lens_t = torch.tensor(lens, dtype=torch.int64, device="cuda")
    if gran == "FP4":
        layer = turbo.modules.Float4GroupedLinear(G, K, N, cache_quantized_weight=cache, device="cuda", dtype=torch.bfloat16)
        op = lambda x, w: turbo.ops.grouped_gemm_fp4(x, w, lens_t, trans_b=True)
        gate = 6
    else:
        cfg = _cfg(m, gran)
        layer = turbo.modules.Float8GroupedLinear(G, K, N, config=cfg, cache_quantized_weight=cache, device="cuda",
                                                  dtype=torch.bfloat16)
        op = lambda x, w: turbo.ops.grouped_gemm_fp8(x, w, lens_t, trans_b=True, config=cfg)
        gate = 22
    with torch.no_grad():
        layer.weight.normal_()
    x = torch.randn(M, K, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    for _ in range(2):
        y = layer(x, lens_t)
        assert torch.equal(y.detach(), op(x.detach(), layer.weight.detach()))
    go = torch.randn_like(y)
    y.backward(go)
    x_ref, w_ref = x.detach().clone().requires_grad_(), layer.weight.detach().clone().requires_grad_()
    offs = [0]
    for n in lens:
        offs.append(offs[-1] + n)
    ref = torch.cat([x_ref[offs[g]:offs[g + 1]].float() @ w_ref[g].float().t() for g in range(G)]).to(torch.bfloat16)
    ref.backward(go)
    assert snr(y, ref) > gate and snr(x.grad, x_ref.grad) > gate
    assert layer.weight.grad is not None
    for g, n in enumerate(lens):
        if n == 0:
            assert float(layer.weight.grad[g].abs().max()) == 0.0
        else:
            assert snr(layer.weight.grad[g], w_ref.grad[g]) > gate


def test_create_quantized_weight_layouts(m):
    from primus_turbo.pytorch.core.quantized_tensor import create_quantized_weight
    w = torch.randn(256, 384, device="cuda", dtype=torch.bfloat16)
    for gran in GRANS:
        cfg = _cfg(m, gran)
        qw, qw_t = create_quantized_weight(w, torch.float8_e4m3fn, cfg, need_weight_transpose_cache=True)
        assert tuple(qw.shape) == (256, 384) and qw_t is not None
        assert snr(qw.dequantize(), w) > 25
        if gran == "TENSORWISE":
            assert tuple(qw_t.shape) == (384, 256)
            assert torch.equal(qw_t.contiguous().qdata.view(torch.uint8), qw.qdata.view(torch.uint8).t().contiguous())
        else:
            assert snr(qw_t.dequantize(), w) > 25
        assert create_quantized_weight(w, torch.float8_e4m3fn, cfg)[1] is None
    qw4, qw4_t = create_quantized_weight(w, torch.float4_e2m1fn_x2, m["Cfg4"](), need_weight_transpose_cache=True)
    assert snr(qw4.dequantize(), w) > 8 and snr(qw4_t.dequantize(), w) > 8
