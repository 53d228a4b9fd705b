"""Run-time plumbing on the GPU: the bounded device wait and its status word, the torch.library operators, torch.compile
around the operators, and invalidation of cached quantized weights after a write that bypasses the version counter."""
import time

import pytest
import torch

pytestmark = pytest.mark.gpu

PT_ERR_TIMEOUT = -4


@pytest.fixture(scope="module")
def nv():
    from primus_turbo.pytorch.kernels import _native
    return _native


def test_bounded_wait_gives_up_and_reports(nv):
    """A wait on a barrier that nothing completes gives up after its limit (1 ms here; the production kernels use 2 s):
    the kernel RETURNS, the status word holds PT_ERR_TIMEOUT and every warp of the CTA saw the abort flag."""
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    observers = torch.zeros(1, dtype=torch.int32, device="cuda")
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    nv.check(nv.lib().pt_wait_probe(1_000_000, nv.ptr(status), nv.ptr(observers), nv.stream(status.device)), "wait_probe")
    torch.cuda.synchronize()
    assert time.perf_counter() - t0 < 2.0, "the probe kernel did not return promptly"
    assert int(status.item()) == PT_ERR_TIMEOUT
    assert int(observers.item()) == 4
    # the context is intact: ordinary work still runs
    assert float(torch.ones(8, device="cuda").sum().item()) == 8.0


def test_status_word_is_surfaced(nv):
    dev = torch.device("cuda", torch.cuda.current_device())
    word = nv.status_word(dev)
    nv.check_status(dev)   # clean to begin with
    # explicit check: raises once, clears the word
    nv.check(nv.lib().pt_wait_probe(200_000, nv.ptr(word), None, nv.stream(dev)), "wait_probe")
    with pytest.raises(RuntimeError, match="gave up waiting"):
        nv.check_status(dev)
    nv.check_status(dev)
    # deferred check: no call waits for the device; the error surfaces at a later operator call
    nv.poll_status(dev)                  # snapshot of a clean word (or nothing, if an earlier snapshot is pending)
    torch.cuda.synchronize()
    nv.poll_status(dev)
    nv.check(nv.lib().pt_wait_probe(200_000, nv.ptr(word), None, nv.stream(dev)), "wait_probe")
    nv.poll_status(dev)                  # may take the snapshot that holds the error
    torch.cuda.synchronize()
    with pytest.raises(RuntimeError, match="gave up waiting"):
        for _ in range(3):
            nv.poll_status(dev)
            torch.cuda.synchronize()
    nv.check_status(dev)                 # cleared by the raise


def test_torch_ops_run_the_same_kernels():
    from primus_turbo.pytorch.core.low_precision import ScalingGranularity as SG
    from primus_turbo.pytorch.kernels.gemm.gemm_fp8_impl import gemm_fp8_impl
    from primus_turbo.pytorch.kernels.quantization import quantization_impl as qi
    g = torch.Generator().manual_seed(0)
    a = torch.randn(256, 512, generator=g).to(torch.bfloat16).cuda()
    b = torch.randn(384, 512, generator=g).to(torch.bfloat16).cuda()
    f8 = torch.float8_e4m3fn
    q1, s1 = torch.ops.primus_turbo.quant_fp8_blockwise_impl(a, f8, 1, 128)
    q2, s2 = qi.quant_fp8_blockwise_impl(a, f8, 1)
    assert torch.equal(q1.view(torch.uint8), q2.view(torch.uint8)) and torch.equal(s1, s2)
    qa, sa = qi.quantize_fp8_tensorwise_impl(a, f8)
    qb, sb = qi.quantize_fp8_tensorwise_impl(b, f8)
    c1 = torch.ops.primus_turbo.gemm_fp8_impl(qa, sa, False, qb, sb, True, torch.bfloat16, False, SG.TENSORWISE.value, 2)
    c2 = gemm_fp8_impl(qa, sa, False, qb, sb, True, torch.bfloat16, False, SG.TENSORWISE)
    assert torch.equal(c1, c2)
    acc = torch.zeros(256, 384, dtype=torch.float32, device="cuda")
    torch.ops.primus_turbo.gemm_fp8_accum_impl(qa, sa, False, qb, sb, True, torch.float32, False, SG.TENSORWISE.value, acc, 2)
    torch.ops.primus_turbo.gemm_fp8_accum_impl(qa, sa, False, qb, sb, True, torch.float32, False, SG.TENSORWISE.value, acc, 2)
    ref = gemm_fp8_impl(qa, sa, False, qb, sb, True, torch.float32, False, SG.TENSORWISE)
    assert torch.allclose(acc, 2 * ref, rtol=1e-6, atol=1e-6)
    h = torch.ops.primus_turbo.gemm_impl(a, False, b, True, torch.bfloat16, False, 2)
    assert torch.allclose(h.float(), a.float() @ b.float().t(), rtol=2e-2, atol=2e-1)


@pytest.mark.parametrize("recipe", ["tensorwise", "mx", "fp4"])
def test_torch_compile_forward_and_backward(recipe):
    """The operators trace and run under torch.compile (forward + backward), as the reference's regression test does
    (tests/pytorch/ops/test_gemm_fp4.py:408-): same values as eager, bit for bit, since the same kernels run."""
    import primus_turbo.pytorch as turbo
    from primus_turbo.pytorch.core.low_precision import (Float4QuantConfig, Float8QuantConfig, Format, ScaleDtype,
                                                         ScalingGranularity)
    if recipe == "tensorwise":
        cfg, op = Float8QuantConfig(format=Format.E4M3, granularity=ScalingGranularity.TENSORWISE), turbo.ops.gemm_fp8
    elif recipe == "mx":
        cfg = Float8QuantConfig(format=Format.E4M3, granularity=ScalingGranularity.MX_BLOCKWISE, scale_dtype=ScaleDtype.E8M0, block_size=32)
        op = turbo.ops.gemm_fp8
    else:
        cfg, op = Float4QuantConfig(), turbo.ops.gemm_fp4
    torch.manual_seed(42)
    a = torch.randn(256, 512, device="cuda", dtype=torch.bfloat16)
    b = torch.randn(256, 512, device="cuda", dtype=torch.bfloat16)
    go = torch.randn(256, 256, device="cuda", dtype=torch.bfloat16)

    def fn(x, y):
        return op(x * 1.0, y, trans_b=True, config=cfg) + 1.0

    def run(f):
        x, y = a.clone().requires_grad_(), b.clone().requires_grad_()
        out = f(x, y)
        out.backward(go)
        return out.detach(), x.grad, y.grad

    eager = run(fn)
    compiled = run(torch.compile(fn))
    for e, c in zip(eager, compiled):
        assert c is not None and torch.isfinite(c.float()).all()
        assert torch.allclose(e.float(), c.float(), rtol=1e-2, atol=1e-2)


def test_quantized_weight_cache_sees_data_writes_after_invalidation():
    """An optimizer that writes parameters through `.data` (main-parameter copies) never bumps the version counter the
    cache is keyed on; `invalidate_quantized_weight_caches()` (or the optimizer step hook that calls it) does."""
    import primus_turbo.pytorch as turbo
    from primus_turbo.pytorch.core.low_precision import Float8QuantConfig, Format, ScalingGranularity
    from primus_turbo.pytorch.modules import invalidate_on_optimizer_step, invalidate_quantized_weight_caches
    torch.manual_seed(3)
    cfg = Float8QuantConfig(format=Format.E4M3, granularity=ScalingGranularity.TENSORWISE)
    lin = turbo.modules.Float8Linear(256, 128, bias=False, config=cfg, cache_quantized_weight=True, device="cuda", dtype=torch.bfloat16)
    x = torch.randn(64, 256, device="cuda", dtype=torch.bfloat16)
    with torch.no_grad():
        y0 = lin(x)
        new_w = torch.randn_like(lin.weight)
        lin.weight.data.copy_(new_w)               # the main-parameter copy of a mixed-precision optimizer
        stale = lin(x)
        assert torch.equal(stale, y0), "expected the cached weight to be served until the cache is invalidated"
        invalidate_quantized_weight_caches()
        fresh = lin(x)
        want = turbo.ops.gemm_fp8(x, new_w, trans_b=True, out_dtype=torch.bfloat16, config=cfg)
        assert torch.equal(fresh, want)
    # the same through an optimizer step hook
    opt = torch.optim.SGD(lin.parameters(), lr=0.0)
    handle = invalidate_on_optimizer_step(opt)
    with torch.no_grad():
        lin(x)
        newer = torch.randn_like(lin.weight)
        lin.weight.data.copy_(newer)
    opt.step()
    with torch.no_grad():
        assert torch.equal(lin(x), turbo.ops.gemm_fp8(x, newer, trans_b=True, out_dtype=torch.bfloat16, config=cfg))
    handle.remove()
