"""BF16 / FP16 gemm and grouped_gemm (the tcgen05 kernels run with 16-bit operands) against an fp32 torch reference:
all transpose combinations, ragged shapes, the CTA-pair path, autograd, zero-length groups, no host synchronisation,
fused main_grad accumulation.  Operator surface: primus_turbo/pytorch/ops/gemm.py and grouped_gemm.py of the
reference; its tests gate on SNR (tests/pytorch/ops/test_gemm.py, test_grouped_gemm.py)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def rel(x, ref):
    x, ref = x.detach().float(), ref.detach().float()
    return float((x - ref).norm() / ref.norm().clamp_min(1e-30))


@pytest.fixture(scope="module")
def turbo():
    import primus_turbo.pytorch as t
    return t


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("M,N,K", [(128, 128, 64), (255, 520, 136), (1024, 384, 4096), (4096, 4096, 1024), (4100, 4360, 520)])
@pytest.mark.parametrize("trans_a,trans_b", [(False, False), (False, True), (True, False), (True, True)])
def test_gemm_matches_fp32_reference(turbo, dtype, M, N, K, trans_a, trans_b):
    torch.manual_seed(0)
    a = torch.randn((K, M) if trans_a else (M, K), device="cuda", dtype=dtype)
    b = torch.randn((N, K) if trans_b else (K, N), device="cuda", dtype=dtype)
    ref = (a.float().t() if trans_a else a.float()) @ (b.float().t() if trans_b else b.float())
    out = turbo.ops.gemm(a, b, trans_a=trans_a, trans_b=trans_b)
    assert out.dtype == dtype and tuple(out.shape) == (M, N)
    assert rel(out, ref) <= (4e-3 if dtype == torch.bfloat16 else 6e-4)   # rounding of the 16-bit output only
    out32 = turbo.ops.gemm(a, b, trans_a=trans_a, trans_b=trans_b, out_dtype=torch.float32)
    assert out32.dtype == torch.float32 and rel(out32, ref) <= 2e-5      # fp32 accumulate in the tensor core (truncating adds), other summation order


def test_gemm_trans_c_and_accumulate(turbo):
    from primus_turbo.pytorch.kernels.gemm.gemm_impl import gemm_accum_impl, gemm_impl
    torch.manual_seed(1)
    a = torch.randn(300, 264, device="cuda", dtype=torch.bfloat16)
    b = torch.randn(200, 264, device="cuda", dtype=torch.bfloat16)
    ref = a.float() @ b.float().t()
    c_t = gemm_impl(a, False, b, True, torch.float32, True)
    assert tuple(c_t.shape) == (200, 300) and rel(c_t, ref.t()) <= 2e-5
    acc = torch.randn(300, 200, device="cuda", dtype=torch.float32)
    want = acc + ref
    gemm_accum_impl(a, False, b, True, torch.float32, False, out=acc)
    assert rel(acc, want) <= 2e-5


@pytest.mark.parametrize("trans_b", [False, True])
def test_gemm_autograd(turbo, trans_b):
    torch.manual_seed(2)
    M, N, K = 512, 384, 256
    a = torch.randn(M, K, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    b = torch.randn((N, K) if trans_b else (K, N), device="cuda", dtype=torch.bfloat16, requires_grad=True)
    a_ref, b_ref = a.detach().float().requires_grad_(), b.detach().float().requires_grad_()
    out = turbo.ops.gemm(a, b, trans_b=trans_b)
    ref = a_ref @ (b_ref.t() if trans_b else b_ref)
    go = torch.randn_like(out)
    out.backward(go)
    ref.backward(go.float())
    assert rel(out, ref) <= 4e-3 and rel(a.grad, a_ref.grad) <= 4e-3 and rel(b.grad, b_ref.grad) <= 4e-3


def _offs(lens):
    lens_t = torch.tensor(lens, dtype=torch.int64, device="cuda")
    offs = torch.zeros(len(lens) + 1, dtype=torch.int64, device="cuda")
    offs[1:] = torch.cumsum(lens_t, 0)
    return lens_t, offs


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("trans_b", [False, True])
@pytest.mark.parametrize("lens", [[100, 0, 300, 29], [1, 300], [0, 0, 5], [512] * 4, [2048, 1024, 3072, 2048]])
def test_grouped_gemm_fwd_bwd_no_host_sync(turbo, dtype, trans_b, lens):
    torch.manual_seed(3)
    lens_t, offs = _offs(lens)
    G, M, K, N = len(lens), int(sum(lens)), 256, 512
    a = torch.randn(M, K, device="cuda", dtype=dtype, requires_grad=True)
    b = (torch.randn((G, N, K) if trans_b else (G, K, N), device="cuda", dtype=dtype) * 0.1).requires_grad_()
    go = torch.randn(M, N, device="cuda", dtype=dtype)
    torch.cuda.synchronize()
    torch.cuda.set_sync_debug_mode("error")
    try:
        out = turbo.ops.grouped_gemm(a, b, lens_t, group_offs=offs, trans_b=trans_b)
        out.backward(go)
    finally:
        torch.cuda.set_sync_debug_mode("default")
    a_ref, b_ref = a.detach().float().requires_grad_(), b.detach().float().requires_grad_()
    o = offs.cpu().tolist()
    ref = torch.cat([a_ref[o[g]:o[g + 1]] @ (b_ref[g].t() if trans_b else b_ref[g]) for g in range(G)])
    ref.backward(go.float())
    tol = 4e-3 if dtype == torch.bfloat16 else 6e-4
    assert tuple(out.shape) == (M, N) and rel(out, ref) <= tol
    assert rel(a.grad, a_ref.grad) <= tol
    assert b.grad.shape == b.shape
    for g, n in enumerate(lens):
        if n == 0:
            assert float(b.grad[g].abs().max()) == 0.0
        else:
            assert rel(b.grad[g], b_ref.grad[g]) <= tol, f"group {g}"


def test_grouped_gemm_fused_main_grad_and_module(turbo):
    torch.manual_seed(4)
    lens = [200, 56, 0, 256]
    lens_t, offs = _offs(lens)
    G, M, K, N = len(lens), int(sum(lens)), 128, 256
    layer = turbo.modules.GroupedLinear(G, K, N, device="cuda", dtype=torch.bfloat16)
    x = torch.randn(M, K, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    go = torch.randn(M, N, device="cuda", dtype=torch.bfloat16)
    y = layer(x, lens_t)
    y.backward(go)
    plain = layer.weight.grad.float().clone()
    w2 = layer.weight.detach().clone().requires_grad_()
    base = torch.randn(G, N, K, device="cuda", dtype=torch.float32)
    w2.main_grad = base.clone()
    w2.grad_added_to_main_grad = False
    y2 = turbo.ops.grouped_gemm(x.detach().requires_grad_(), w2, lens_t, trans_b=True, fuse_bgrad_accum_pattern="megatron")
    assert torch.equal(y2, y)
    y2.backward(go)
    assert w2.grad_added_to_main_grad
    assert rel(w2.main_grad - base, plain) <= 4e-3
