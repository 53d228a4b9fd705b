"""MoE token permutation: the CUDA kernels against the reference's own unfused definition, which is a composition of torch
indexing calls (primus_turbo/pytorch/ops/moe/permutation.py:344-377,440-): masked_select / index_select / index_add.  Copies
are bit exact; the weighted sums are compared to fp32 arithmetic in the same order."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _routing(T, E, topk, seed, empty_expert=None):
    g = torch.Generator().manual_seed(seed)
    scores = torch.rand(T, E, generator=g)
    if empty_expert is not None:
        scores[:, empty_expert] = -1.0
    idx = scores.topk(topk, dim=1).indices
    rm = torch.zeros(T, E, dtype=torch.bool)
    rm.scatter_(1, idx, True)
    probs = torch.rand(T, E, generator=g) * rm
    return rm.cuda(), probs.float().cuda()


def _ref_permute(inp, rm, probs):
    """The unfused reference: expert-major order, tokens ascending inside an expert."""
    T, E = rm.shape
    rmt = rm.bool().T.contiguous()
    token_indices = torch.arange(T, device=rm.device).unsqueeze(0).expand(E, -1)
    sorted_indices = token_indices.masked_select(rmt)
    permuted_probs = probs.T.contiguous().masked_select(rmt) if probs is not None else None
    return inp.index_select(0, sorted_indices), permuted_probs, sorted_indices, rmt.sum(dim=1)


@pytest.mark.parametrize("T,E,topk,H", [(64, 8, 2, 256), (1000, 64, 8, 1024), (4096, 256, 8, 7168), (17, 3, 1, 64)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("map_dtype", [torch.bool, torch.int32])
def test_permute_and_unpermute_match_the_unfused_definition(T, E, topk, H, dtype, map_dtype):
    import primus_turbo.pytorch as turbo
    rm, probs = _routing(T, E, topk, seed=T + E, empty_expert=1 if E > 2 else None)
    g = torch.Generator().manual_seed(7)
    x = torch.randn(T, H, generator=g).to(dtype).cuda()
    out, pprobs, row_id_map, tpe = turbo.ops.token_permute(x, -1, probs=probs, routing_map=rm.to(map_dtype), return_tokens_per_expert=True)
    want, want_probs, sorted_indices, want_tpe = _ref_permute(x, rm, probs)
    assert torch.equal(out, want) and torch.equal(pprobs, want_probs)
    assert torch.equal(tpe, want_tpe.to(torch.int64))
    assert tuple(row_id_map.shape) == (T, 2 * E + 1) and int(row_id_map[:, -1].sum()) == T * topk
    # unpermute without probabilities: plain sum of a token's rows (fp32 accumulation, expert order)
    back = turbo.ops.token_unpermute(out, row_id_map, restore_shape=x.shape)
    ref = torch.zeros(T, H, dtype=torch.float32, device="cuda").index_add_(0, sorted_indices, want.float())
    tol = dict(rtol=0, atol=0) if dtype == torch.float32 and topk == 1 else dict(rtol=1e-2 if dtype == torch.bfloat16 else 1e-6, atol=1e-2 if dtype == torch.bfloat16 else 1e-5)
    assert torch.allclose(back.float(), ref, **tol)
    # weighted
    y = torch.randn(out.shape, generator=g).to(dtype).cuda()
    merged = turbo.ops.token_unpermute(y, row_id_map, merging_probs=probs, restore_shape=x.shape)
    ref = torch.zeros(T, H, dtype=torch.float32, device="cuda").index_add_(0, sorted_indices, y.float() * want_probs.unsqueeze(-1))
    assert torch.allclose(merged.float(), ref, rtol=1e-2 if dtype == torch.bfloat16 else 1e-5, atol=1e-2 if dtype == torch.bfloat16 else 1e-5)


def test_autograd_of_permute_and_unpermute():
    import primus_turbo.pytorch as turbo
    T, E, topk, H = 512, 16, 4, 512
    rm, probs = _routing(T, E, topk, seed=3)
    g = torch.Generator().manual_seed(9)
    x = torch.randn(T, H, generator=g).float().cuda().requires_grad_()
    p = probs.clone().requires_grad_()
    out, pprobs, row_id_map, _ = turbo.ops.token_permute(x, T * topk, probs=p, routing_map=rm)
    y = turbo.ops.token_unpermute(out * 2.0, row_id_map, merging_probs=p, restore_shape=x.shape)
    loss = (y * torch.arange(H, device="cuda").float()).sum() + (pprobs * 3.0).sum()
    loss.backward()
    # the same with torch indexing
    x2, p2 = x.detach().clone().requires_grad_(), probs.clone().requires_grad_()
    rmt = rm.T.contiguous()
    sorted_indices = torch.arange(T, device="cuda").unsqueeze(0).expand(E, -1).masked_select(rmt)
    out2 = x2.index_select(0, sorted_indices)
    pp2 = p2.T.contiguous().masked_select(rmt)
    y2 = torch.zeros(T, H, device="cuda").index_add(0, sorted_indices, out2 * 2.0 * pp2.unsqueeze(-1))
    loss2 = (y2 * torch.arange(H, device="cuda").float()).sum() + (pp2 * 3.0).sum()
    loss2.backward()
    assert torch.allclose(y, y2, rtol=1e-5, atol=1e-4)
    assert torch.allclose(x.grad, x2.grad, rtol=1e-5, atol=1e-3)
    assert torch.allclose(p.grad, p2.grad, rtol=1e-4, atol=1e-1)


def test_permute_feeds_the_grouped_gemm():
    """The permuted rows and tokens_per_expert are exactly what grouped_gemm_fp8 takes: one MoE expert layer end to end."""
    import primus_turbo.pytorch as turbo
    from primus_turbo.pytorch.core.low_precision import Float8QuantConfig, Format, ScalingGranularity
    T, E, topk, H, F = 1024, 8, 2, 512, 768
    rm, probs = _routing(T, E, topk, seed=5)
    x = torch.randn(T, H, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(E, F, H, device="cuda", dtype=torch.bfloat16) * 0.05
    cfg = Float8QuantConfig(format=Format.E4M3, granularity=ScalingGranularity.BLOCKWISE, block_size=128)
    xp, pp, row_id_map, tpe = turbo.ops.token_permute(x, T * topk, probs=probs, routing_map=rm, return_tokens_per_expert=True)
    h = turbo.ops.grouped_gemm_fp8(xp, w, tpe, trans_b=True, config=cfg)
    y = turbo.ops.token_unpermute(h, row_id_map, merging_probs=probs, restore_shape=torch.Size((T, F)))
    ref = torch.zeros(T, F, device="cuda")
    for e in range(E):
        sel = rm[:, e]
        ref[sel] += (x[sel].float() @ w[e].float().t()) * probs[sel, e].unsqueeze(-1)
    err = (y.float() - ref).norm() / ref.norm()
    assert float(err) < 0.08


@pytest.mark.parametrize("T,E,topk", [(1, 1, 1), (33, 5, 2), (1000, 40, 3), (16384, 256, 8), (2050, 1024, 4), (300, 1100, 2)])
@pytest.mark.parametrize("map_dtype", [torch.bool, torch.int32, torch.int64])
def test_row_id_map_layout(T, E, topk, map_dtype):
    """row_id_map [T, 2E + 1] against its definition: per token the destination rows of its routed experts in ascending
    expert order, the expert ids, and their number; destinations follow the expert-major order of the unfused reference.
    E = 1100 takes the per-expert-column kernels, the others the row-major ones."""
    from primus_turbo.pytorch.kernels.moe import permutation_impl as pm
    rm, _ = _routing(T, E, topk, seed=7 * T + E, empty_expert=1 if E > 2 else None)
    row_id_map, tpe = pm.make_row_id_map(rm.to(map_dtype), T, E)
    rmt = rm.T.contiguous()
    assert torch.equal(tpe.cpu(), rmt.sum(dim=1).cpu())
    # destination of (e, t) in expert-major order = exclusive rank of the pair among the routed pairs
    flat = rmt.reshape(-1).to(torch.int64)
    dest = (flat.cumsum(0) - flat).reshape(E, T).T          # [T, E]
    m = row_id_map.cpu()
    n = m[:, 2 * E]
    assert torch.equal(n, rm.sum(dim=1).cpu().to(m.dtype))
    rm_c, dest_c = rm.cpu(), dest.cpu()
    for t in (0, T // 2, T - 1):
        es = torch.nonzero(rm_c[t]).flatten()
        k = len(es)
        assert torch.equal(m[t, E:E + k].long(), es) and torch.equal(m[t, :k].long(), dest_c[t, es])
        assert (m[t, k:E] == -1).all() and (m[t, E + k:2 * E] == -1).all()
    # every destination row is used exactly once
    used = m[:, :E][m[:, :E] >= 0]
    assert used.numel() == int(flat.sum()) and torch.equal(used.sort().values, torch.arange(used.numel(), dtype=used.dtype))
