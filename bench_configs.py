"""Workloads of the five benchmark configurations and the per-configuration measurements `bench.py` prints
beside its headline: quantizer GB/s, dense forward / dgrad / wgrad, grouped forward / dgrad / wgrad.

Everything here calls the same `*_impl` functions the operators call (one extern "C" entry each).  Shapes:

  C2  Llama-3-8B MLP      M=8192   K=4096  N=14336                      rowwise and 128-blockwise FP8
  C3  Llama-3-70B FFN     M=16384  K=8192  N=28672                      MXFP8, forward + wgrad
  C4  DeepSeek-V3 MoE     256 experts, 131072 rows, 7168 -> 4096 and 2048 -> 7168, Zipf(1.1) group lengths
  C5  Mixtral-8x7B MoE    8 experts, 65536 rows, 4096 -> 14336, Dirichlet(0.3) group lengths, MXFP4

The group-length generators are shared with tests/test_configs_gpu.py so that tests and measurements see the same
ragged layouts.  Large operands are drawn with the device generator (seeded): 15 GB of weights do not fit a host
generator's patience; the parity tests download the rows they compare.
"""
import os
import statistics

import numpy as np
import torch

C2 = dict(M=8192, K=4096, N=14336, seed=1)
C3 = dict(M=16384, K=8192, N=28672, seed=2)
C4 = dict(G=256, rows=131072, hidden=7168, inter2=4096, inter=2048, seed=3)
C5 = dict(G=8, rows=65536, hidden=4096, ffn=14336, seed=4)


# ---------------------------------------------------------------------------------------------- group lengths
def zipf_group_lens(G=256, rows=131072, s=1.1, seed=3, empty=4):
    """Multinomial(rows, p) with p_i proportional to (i + 1)^-s, randomly permuted; the `empty` least loaded experts
    are emptied and their rows given to the most loaded one, so that the layout always has empty groups."""
    rng = np.random.default_rng(seed)
    p = np.arange(1, G + 1, dtype=np.float64) ** -s
    p = p[rng.permutation(G)]
    p /= p.sum()
    lens = rng.multinomial(rows, p).astype(np.int64)
    order = np.argsort(lens, kind="stable")
    lens[order[-1]] += lens[order[:empty]].sum()
    lens[order[:empty]] = 0
    assert lens.sum() == rows
    return lens


def dirichlet_group_lens(G=8, rows=65536, alpha=0.3, seed=4):
    """round(rows * Dirichlet(alpha)) with the remainder on the last group."""
    rng = np.random.default_rng(seed)
    frac = rng.dirichlet(alpha * np.ones(G))
    lens = np.floor(frac * rows).astype(np.int64)
    lens[-1] = rows - lens[:-1].sum()
    assert lens.min() >= 0 and lens.sum() == rows
    return lens


def offsets_of(lens, device):
    lens_t = torch.as_tensor(np.asarray(lens), dtype=torch.int64, device=device)
    offs = torch.zeros(lens_t.numel() + 1, dtype=torch.int64, device=device)
    offs[1:] = torch.cumsum(lens_t, 0)
    return lens_t, offs


def randn_bf16(shape, std, seed, device):
    g = torch.Generator(device=device).manual_seed(seed)
    x = torch.empty(shape, dtype=torch.bfloat16, device=device)
    x.normal_(0.0, std, generator=g)
    return x


# ---------------------------------------------------------------------------------------------- timing
def time_cuda(fn, iters=20, warmup=3):
    """Median CUDA-event time of one call in ms (events on the current stream, one synchronise per call)."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1))
    return statistics.median(ts)


def time_cuda_rotating(fns, rounds=12, warmup=2):
    """Median device time of one call when the calls cycle through `fns` (same kernel, different input buffers whose
    sum exceeds L2, so that no call finds its input cached).  One round of all calls is captured in a CUDA graph and
    the replays are timed with events: the kernels run back to back as they do inside a training step, and the host
    cost of the Python wrappers (about as long as a 30 us kernel) stays out of the figure.  Falls back to timing
    eager calls if the capture fails."""
    n = len(fns)
    for _ in range(warmup):
        for f in fns:
            f()
    torch.cuda.synchronize()
    replay = None
    # Captured launches of the persistent quantizers normally keep the static tile schedule (a replay could overlap
    # another launch that holds the same counter slot); this graph is the only work on the device, so the dynamic
    # schedule the eager launches of a training step get is allowed into it.
    before = os.environ.get("PT_TILE_SCHED_IN_GRAPHS")
    os.environ["PT_TILE_SCHED_IN_GRAPHS"] = "1"
    try:
        graph = torch.cuda.CUDAGraph()
        keep = []
        with torch.cuda.graph(graph):
            for f in fns:
                keep.append(f())     # outputs stay alive: every call writes its own buffers
        replay = graph.replay
    except Exception:  # noqa: BLE001
        torch.cuda.synchronize()
    finally:
        if before is None:
            os.environ.pop("PT_TILE_SCHED_IN_GRAPHS", None)
        else:
            os.environ["PT_TILE_SCHED_IN_GRAPHS"] = before
    if replay is None:
        def replay():
            for f in fns:
                f()
    replay()
    torch.cuda.synchronize()
    ts = []
    for _ in range(rounds):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        replay()
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1) / n)
    return statistics.median(ts)


def _tensor_rec(flops, ms, peaks, kind, kernel):
    """TFLOP/s record of a GEMM timed alone in a short loop: the burst figure is the denominator (x2 for FP8, x4 for
    FP4 over the measured bf16 GEMM), the sustained one is printed beside it."""
    mult = {"fp8": 2.0, "fp4": 4.0, "bf16": 1.0}[kind]
    tf = flops / (ms / 1e3) / 1e12
    return {"ms": ms, "tflops": tf, "roofline": {"bound": "tensor", "achieved": tf, "peak": mult * peaks["bf16_burst"],
            "frac": tf / (mult * peaks["bf16_burst"]), "frac_of_sustained": tf / (mult * peaks["bf16_sustained"]),
            "frac_of_nominal": tf / (2250.0 * mult), "unit": "TFLOP/s", "kernel": kernel}}


def _hbm_rec(nbytes, ms, peaks, kernel):
    gbs = nbytes / (ms / 1e3) / 1e9
    return {"ms": ms, "bytes": nbytes, "gbs": gbs, "roofline": {"bound": "hbm", "achieved": gbs, "peak": peaks["hbm_gbs"],
            "frac": gbs / peaks["hbm_gbs"], "unit": "GB/s", "kernel": kernel}}


# ---------------------------------------------------------------------------------------------- quantizers
def quantize_records(dev, peaks, copies=4):
    """One entry per quantizer on the tensor its configuration gives it; algorithmic bytes = input + outputs + scales."""
    from primus_turbo.pytorch.core.low_precision import ScalingRecipe as SR
    from primus_turbo.pytorch.kernels.quantization import quantization_impl as qi
    f8, f5, f4 = torch.float8_e4m3fn, torch.float8_e5m2, torch.float4_e2m1fn_x2
    out = {}
    M, K, N = C2["M"], C2["K"], C2["N"]

    def act(seed):
        x = randn_bf16((M, K), 1.0, seed, dev)
        mask = torch.rand((M, K), device=dev, generator=torch.Generator(device=dev).manual_seed(seed + 100)) < 0.001
        return torch.where(mask, x * 50, x)

    acts = [act(10 + i) for i in range(copies)]
    wts = [randn_bf16((N, K), 0.02, 20 + i, dev) for i in range(copies)]
    two_d = SR(use_2d_block=True)

    def run(name, fns, nbytes, kernel):
        out[name] = _hbm_rec(nbytes, time_cuda_rotating(fns), peaks, kernel)

    e, ew = M * K, N * K
    run("tensorwise_act_8192x4096", [lambda x=x: qi.quantize_fp8_tensorwise_impl(x, f8) for x in acts], 2 * 2 * e + e + 4,
        "amax_flat_kernel + cast_flat_kernel")
    run("rowwise_act_8192x4096", [lambda x=x: qi.quantize_fp8_rowwise_impl(x, f8, -1) for x in acts], 3 * e + 4 * M,
        "rowwise_last_axis_kernel")
    run("rowwise_other_axis_act_8192x4096", [lambda x=x: qi.quantize_fp8_rowwise_impl(x, f8, -2) for x in acts], 5 * e + 4 * K,
        "amax_cols_kernel + cast_cols_kernel")
    run("blockwise_row_act_8192x4096", [lambda x=x: qi.quant_fp8_blockwise_impl(x, f8, 1) for x in acts], 3 * e + 4 * e // 128,
        "blockwise_tma_kernel<ROW>")
    run("blockwise_dual_act_8192x4096", [lambda x=x: qi.quant_fp8_blockwise_dual_impl(x, f8) for x in acts], 4 * e + 8 * e // 128,
        "blockwise_split_kernel")
    run("blockwise_weight_14336x4096", [lambda w=w: qi.quant_fp8_blockwise_for_weight_impl(w, f8) for w in wts],
        3 * ew + 4 * ew // 16384, "blockwise_tma_kernel<WEIGHT>")
    run("mxfp8_row_act_8192x4096", [lambda x=x: qi.quantize_mxfp8_impl(x, f8, 1, 32) for x in acts], 3 * e + e // 32,
        "mx_quant_tma_kernel<row>")
    run("mxfp8_dual_act_8192x4096", [lambda x=x: qi.quantize_mxfp8_impl(x, f8, None, 32, True) for x in acts],
        2 * e + 2 * (e + e // 32), "mx_quant_split_kernel<e4m3>")
    run("mxfp8_dual_2d_weight_14336x4096", [lambda w=w: qi.quantize_mxfp8_impl(w, f8, None, 32, True, two_d, two_d) for w in wts],
        2 * ew + 2 * (ew + ew // 32), "mx_quant_split_kernel<e4m3, 2-D>")
    run("mxfp4_dual_act_8192x4096", [lambda x=x: qi.quantize_mxfp4_impl(x, f4, None, 32, True) for x in acts],
        2 * e + 2 * (e // 2 + e // 32), "mx_quant_split_kernel<e2m1>")
    del wts
    # C3: dual MX quantization of the 16384 x 8192 activation (the transposed copy feeds the wgrad)
    a3 = [randn_bf16((C3["M"], C3["K"]), 1.0, 30 + i, dev) for i in range(2)]
    e3 = C3["M"] * C3["K"]
    run("mxfp8_dual_act_16384x8192", [lambda x=x: qi.quantize_mxfp8_impl(x, f8, None, 32, True) for x in a3],
        2 * e3 + 2 * (e3 + e3 // 32), "mx_quant_split_kernel<e4m3>")
    del a3
    # C4: segment-M row + column quantization of 32768 of the routed rows (hidden 7168), Zipf lengths of 64 experts
    lens = zipf_group_lens(64, 32768, seed=C4["seed"])
    lens_t, offs = offsets_of(lens, dev)
    xs = [randn_bf16((32768, C4["hidden"]), 1.0, 40 + i, dev) for i in range(2)]
    e4 = 32768 * C4["hidden"]
    e4_pad = int(((lens + 127) // 128 * 128).sum()) * C4["hidden"]
    run("blockwise_segment_m_32768x7168_g64", [lambda x=x: qi.quant_fp8_blockwise_segment_m_row_col_impl(x, f8, 128, lens_t, offs) for x in xs],
        2 * e4 + e4 + e4_pad + 4 * e4 // 128 + 4 * e4_pad // 128, "blockwise_split_kernel<segment-M>")
    del xs
    # C5: grouped MXFP4 dual quantization (row copy plain, transposed copy with the 16-point Hadamard transform)
    lens5 = dirichlet_group_lens(C5["G"], C5["rows"], seed=C5["seed"])
    lens5_t, offs5 = offsets_of(lens5, dev)
    x5 = [randn_bf16((C5["rows"], C5["hidden"]), 1.0, 50 + i, dev) for i in range(2)]
    e5 = C5["rows"] * C5["hidden"]
    e5_pad = int(((lens5 + 255) // 256 * 256).sum()) * C5["hidden"]
    run("grouped_mxfp4_dual_rht_65536x4096_g8",
        [lambda x=x: qi.grouped_quantize_mxfp4_impl(x, f4, None, 32, lens5_t, offs5, with_trans=True, scaling_recipe=SR(),
                                                    scaling_recipe_for_trans=SR(use_rht=True)) for x in x5],
        2 * e5 + (e5 // 2 + e5 // 32) + (e5_pad // 2 + e5_pad // 32), "mx_quant_split_kernel<e2m1, grouped, Hadamard columns>")
    run("grouped_mxfp8_dual_65536x4096_g8",
        [lambda x=x: qi.grouped_quantize_mxfp8_impl(x, f8, None, 32, lens5_t, offs5, with_trans=True) for x in x5],
        2 * e5 + 2 * (e5 + e5 // 32), "mx_quant_split_kernel<e4m3, grouped>")
    del x5
    # The step between the two grouped GEMMs of an expert MLP (C4: intermediate 2048, 32768 of the routed rows): SwiGLU with
    # probabilities and the dual MX quantization of its result, as one kernel and as two.  Algorithmic bytes of the one-pass
    # form: the [rows, 2 I] input + both copies with scales; the two-kernel form also writes and re-reads [rows, I] bf16.
    rows, inter = 32768, C4["inter"]
    xg = [randn_bf16((rows, 2 * inter), 1.0, 60 + i, dev) for i in range(3)]
    probs = torch.rand(rows, device=dev, generator=torch.Generator(device=dev).manual_seed(61))
    eo = rows * inter
    for nm, od, ob in (("mxfp8", f8, 2 * (eo + eo // 32)), ("mxfp4", f4, 2 * (eo // 2 + eo // 32))):
        run(f"swiglu_{nm}_dual_one_pass_{rows}x{inter}", [lambda x=x: qi.glu_quantize_mx_impl(x, probs, None, "silu", od, fused=True) for x in xg],
            4 * eo + 4 * rows + ob, "mx_quant_split_kernel<SwiGLU prologue>")
        run(f"swiglu_{nm}_dual_two_kernels_{rows}x{inter}", [lambda x=x: qi.glu_quantize_mx_impl(x, probs, None, "silu", od, fused=False) for x in xg],
            4 * eo + 4 * rows + ob, "glu_fwd_kernel + mx_quant_split_kernel (same algorithmic bytes counted; moves 4 more bytes per element)")
    for fused, nm in ((True, "one_pass"), (False, "two_kernels")):   # the forward-only form: row-wise copy alone
        run(f"swiglu_mxfp8_row_{nm}_{rows}x{inter}", [lambda x=x: qi.glu_quantize_mx_row_impl(x, probs, None, "silu", f8, fused=fused) for x in xg],
            4 * eo + 4 * rows + eo + eo // 32, "glu_mx_row_kernel" if fused else "glu_fwd_kernel + mx_quant_tma_kernel (same algorithmic bytes counted)")
    del xg
    # RMSNorm feeding an MX GEMM (C2's activation): statistics pass + normalising quantizer against rmsnorm + quantizer
    gam = randn_bf16((K,), 1.0, 62, dev)
    for fused, nm in ((True, "one_pass"), (False, "two_kernels")):
        run(f"rmsnorm_mxfp8_dual_{nm}_8192x4096", [lambda x=x: qi.rmsnorm_quantize_mx_impl(x, gam, 1e-6, False, f8, fused=fused) for x in acts],
            2 * e + 2 * (e + e // 32) + 4 * M, "rmsnorm_fwd_kernel<statistics> + mx_quant_split_kernel<RMSNorm prologue>" if fused
            else "rmsnorm_fwd_kernel + mx_quant_split_kernel")
    # the forward-only form: RMSNorm and the row-wise MX copy alone
    for fused, nm in ((True, "one_pass"), (False, "two_kernels")):
        run(f"rmsnorm_mxfp8_row_{nm}_8192x4096", [lambda x=x: qi.rmsnorm_quantize_mx_row_impl(x, gam, 1e-6, False, f8, fused=fused) for x in acts],
            2 * e + (e + e // 32) + 4 * M, "rmsnorm_mx_row_kernel" if fused else "rmsnorm_fwd_kernel + mx_quant_tma_kernel (same algorithmic bytes counted)")
    return out


# ---------------------------------------------------------------------------------------------- dense C2 backward
def dense_bwd_c2(dev, peaks):
    """dgrad [8192 x 14336] -> [8192 x 4096] and wgrad -> [14336 x 4096] of the C2 linear, rowwise and blockwise,
    e4m3 forward operands and e5m2 gradients, GEMM kernels timed on pre-quantized operands (quantizers have their own
    records)."""
    from primus_turbo.pytorch.core.low_precision import ScalingGranularity as SG, ScalingRecipe as SR
    from primus_turbo.pytorch.kernels.gemm.gemm_fp8_impl import gemm_fp8_impl
    from primus_turbo.pytorch.kernels.quantization import quantization_impl as qi
    f8, f5 = torch.float8_e4m3fn, torch.float8_e5m2
    M, K, N = C2["M"], C2["K"], C2["N"]
    x = randn_bf16((M, K), 1.0, 61, dev)
    w = randn_bf16((N, K), 0.02, 62, dev)
    dy = randn_bf16((M, N), 1e-3, 63, dev)
    flops = 2.0 * M * N * K
    out = {}
    # rowwise: dgrad = g(row scales) . w_t(col-axis scales);  wgrad = x_t^T . g_t  (scales along the tokens)
    g_q, g_s = qi.quantize_fp8_rowwise_impl(dy, f5, -1)
    wt_q, wt_s = qi.quantize_fp8_rowwise_impl(w, f8, -2)
    out["rowwise_dgrad"] = _tensor_rec(flops, time_cuda(lambda: gemm_fp8_impl(g_q, g_s, False, wt_q, wt_s, False, torch.bfloat16, False, SG.ROWWISE)),
                                       peaks, "fp8", "gemm_fp8_pair_kernel<ROW> (+ transposed weight copy)")
    xt_q, xt_s = qi.quantize_fp8_rowwise_impl(x, f8, -2)
    gt_q, gt_s = qi.quantize_fp8_rowwise_impl(dy, f5, -2)
    out["rowwise_wgrad"] = _tensor_rec(flops, time_cuda(lambda: gemm_fp8_impl(xt_q, xt_s, True, gt_q, gt_s, False, torch.bfloat16, True, SG.ROWWISE)),
                                       peaks, "fp8", "gemm_fp8_pair_kernel<ROW> (+ transposed operand copies)")
    del g_q, wt_q, xt_q, gt_q
    # blockwise: operands of the backward GEMMs are the forward's tensors read MN-major in place
    _, _, a_col, a_col_s = qi.quant_fp8_blockwise_dual_impl(x, f8)
    b_q, b_s = qi.quant_fp8_blockwise_for_weight_impl(w, f8)
    g_row, g_row_s, g_col, g_col_s = qi.quant_fp8_blockwise_dual_impl(dy, f5)
    out["blockwise_dgrad"] = _tensor_rec(flops, time_cuda(lambda: gemm_fp8_impl(g_row, g_row_s, False, b_q, b_s, False, torch.bfloat16, False, SG.BLOCKWISE)),
                                         peaks, "fp8", "gemm_fp8_blockwise_kernel")
    out["blockwise_wgrad"] = _tensor_rec(flops, time_cuda(lambda: gemm_fp8_impl(a_col, a_col_s, True, g_col, g_col_s, False, torch.bfloat16, True, SG.BLOCKWISE)),
                                         peaks, "fp8", "gemm_fp8_blockwise_kernel")
    return out


# ---------------------------------------------------------------------------------------------- C3 (MXFP8 70B FFN)
def mx_c3(dev, peaks, n_lo=0, n_hi=None):
    """Forward and wgrad of the 16384 x 28672 x 8192 MXFP8 linear restricted to output columns [n_lo, n_hi) (the whole
    layer by default; one rank's shard in the N-sharded run).  The wgrad contracts the transposed MX copies."""
    from primus_turbo.pytorch.core.low_precision import ScalingGranularity as SG, ScalingRecipe as SR
    from primus_turbo.pytorch.kernels.gemm.gemm_fp8_impl import gemm_fp8_impl
    from primus_turbo.pytorch.kernels.quantization import quantization_impl as qi
    f8, f5 = torch.float8_e4m3fn, torch.float8_e5m2
    M, K, N = C3["M"], C3["K"], C3["N"]
    n_hi = N if n_hi is None else n_hi
    n = n_hi - n_lo
    x = randn_bf16((M, K), 1.0, 71, dev)
    w = randn_bf16((N, K), 0.01, 72, dev)[n_lo:n_hi].contiguous()
    dy = randn_bf16((M, n), 1e-3, 73 + n_lo, dev)
    two_d = SR(use_2d_block=True)
    a_row, a_row_s, a_col, a_col_s = qi.quantize_mxfp8_impl(x, f8, None, 32, True)
    b_row, b_row_s, _, _ = qi.quantize_mxfp8_impl(w, f8, None, 32, True, two_d, two_d)
    _, _, g_col, g_col_s = qi.quantize_mxfp8_impl(dy, f5, None, 32, True)
    del x, w, dy
    flops = 2.0 * M * n * K
    out = {"columns": [n_lo, n_hi]}
    out["fwd"] = _tensor_rec(flops, time_cuda(lambda: gemm_fp8_impl(a_row, a_row_s, False, b_row, b_row_s, True, torch.bfloat16, False, SG.MX_BLOCKWISE)),
                             peaks, "fp8", "gemm_fp8_pair_kernel<MX>")
    out["wgrad"] = _tensor_rec(flops, time_cuda(lambda: gemm_fp8_impl(g_col, g_col_s, False, a_col, a_col_s, True, torch.bfloat16, False, SG.MX_BLOCKWISE)),
                               peaks, "fp8", "gemm_fp8_pair_kernel<MX>")
    return out


# ---------------------------------------------------------------------------------------------- C4 (blockwise MoE)
def grouped_blockwise_c4(dev, peaks, g_lo=0, g_hi=None, projections=("gate_up", "down"), iters=8, lens=None):
    """Blockwise-FP8 grouped forward / dgrad / wgrad over experts [g_lo, g_hi) of the 256 (all by default; one rank's
    experts in the expert-sharded run) with the rows routed to them (`lens`: this rank's share of each of them, when
    popular experts are split between ranks)."""
    from primus_turbo.pytorch.core.low_precision import ScalingGranularity as SG
    from primus_turbo.pytorch.kernels.grouped_gemm import grouped_gemm_fp8_impl as ggi
    from primus_turbo.pytorch.kernels.quantization import quantization_impl as qi
    f8, f5 = torch.float8_e4m3fn, torch.float8_e5m2
    lens_all = zipf_group_lens(C4["G"], C4["rows"], seed=C4["seed"])
    g_hi = C4["G"] if g_hi is None else g_hi
    lens = lens_all[g_lo:g_hi] if lens is None else np.asarray(lens, dtype=np.int64)
    rows, G = int(lens.sum()), int(g_hi - g_lo)
    lens_t, offs = offsets_of(lens, dev)
    out = {"experts": [int(g_lo), int(g_hi)], "rows": rows, "empty_groups": int((lens == 0).sum()), "max_group": int(lens.max())}
    shapes = {"gate_up": (C4["inter2"], C4["hidden"]), "down": (C4["hidden"], C4["inter"])}
    for name in projections:
        N, K = shapes[name]
        x = randn_bf16((max(rows, 1), K), 1.0, 81 + g_lo, dev)[:rows]
        dy = randn_bf16((max(rows, 1), N), 1e-3, 82 + g_lo, dev)[:rows]
        w = randn_bf16((G, N, K), 0.02, 83 + g_lo, dev)
        a_row, a_col, a_s_row, a_s_col, plens, poffs = qi.quant_fp8_blockwise_segment_m_row_col_impl(x, f8, 128, lens_t, offs)
        w_q, w_s = qi.quant_fp8_blockwise_for_weight_impl(w, f8)
        g_row, g_col, g_s_row, g_s_col, _, _ = qi.quant_fp8_blockwise_segment_m_row_col_impl(dy, f5, 128, lens_t, offs)
        del x, dy, w
        flops = 2.0 * rows * N * K
        rec = {}
        rec["fwd"] = _tensor_rec(flops, time_cuda(lambda: ggi.grouped_gemm_fp8_impl(a_row, w_q, a_s_row, w_s, lens_t, offs, False, True, torch.bfloat16, SG.BLOCKWISE), iters),
                                 peaks, "fp8", "gemm_fp8_blockwise_kernel (grouped)")
        rec["dgrad"] = _tensor_rec(flops, time_cuda(lambda: ggi.grouped_gemm_fp8_impl(g_row, w_q, g_s_row, w_s, lens_t, offs, False, False, torch.bfloat16, SG.BLOCKWISE), iters),
                                   peaks, "fp8", "gemm_fp8_blockwise_kernel (grouped, MN-major weight)")
        rec["wgrad"] = _tensor_rec(flops, time_cuda(lambda: ggi.grouped_gemm_fp8_variable_k_impl(a_col, g_col, a_s_col, g_s_col, plens, poffs, True, False, True, torch.bfloat16, SG.BLOCKWISE), max(3, iters // 2)),
                                   peaks, "fp8", "gemm_fp8_blockwise_kernel (variable K)")
        rec["wgrad"]["output_bytes"] = 2 * G * N * K
        out[name] = rec
        del a_row, a_col, w_q, g_row, g_col
        torch.cuda.empty_cache()
    return out


# ---------------------------------------------------------------------------------------------- C5 (MXFP4 MoE)
def grouped_mxfp4_c5(dev, peaks, lens=None, iters=8):
    """MXFP4 grouped forward / dgrad / wgrad, 8 experts 4096 -> 14336; `lens` overrides the Dirichlet group lengths
    (the tokens-per-expert sweep passes balanced ones)."""
    from primus_turbo.pytorch.core.low_precision import ScalingRecipe as SR
    from primus_turbo.pytorch.kernels.grouped_gemm import grouped_gemm_fp4_impl as gg4
    from primus_turbo.pytorch.kernels.quantization import quantization_impl as qi
    f4 = torch.float4_e2m1fn_x2
    G, K, N = C5["G"], C5["hidden"], C5["ffn"]
    lens = dirichlet_group_lens(G, C5["rows"], seed=C5["seed"]) if lens is None else np.asarray(lens, dtype=np.int64)
    rows = int(lens.sum())
    lens_t, offs = offsets_of(lens, dev)
    x = randn_bf16((rows, K), 1.0, 91, dev)
    dy = randn_bf16((rows, N), 1.0, 92, dev)
    w = randn_bf16((G, N, K), 0.02, 93, dev)
    rht = SR(use_rht=True)
    two_d = SR(use_2d_block=True)
    a_row, a_s_row, a_col, a_s_col, _, orow, lcol, ocol = qi.grouped_quantize_mxfp4_impl(x, f4, None, 32, lens_t, offs, with_trans=True,
                                                                                         scaling_recipe=SR(), scaling_recipe_for_trans=rht)
    w_row, w_s_row, w_col, w_s_col = qi.quantize_mxfp4_impl(w, f4, None, 32, with_trans=True, scaling_recipe=two_d, scaling_recipe_for_trans=two_d)
    g_row, g_s_row, g_col, g_s_col, _, orow2, _, _ = qi.grouped_quantize_mxfp4_impl(dy, f4, None, 32, lens_t, offs, with_trans=True,
                                                                                    scaling_recipe=SR(), scaling_recipe_for_trans=rht)
    del x, dy, w
    flops = 2.0 * rows * N * K
    out = {"group_lens": [int(v) for v in lens]}
    out["fwd"] = _tensor_rec(flops, time_cuda(lambda: gg4.grouped_gemm_fp4_impl(a_row, w_row, a_s_row, w_s_row, lens_t, orow, out_dtype=torch.bfloat16, group_offs_out=offs), iters),
                             peaks, "fp4", "gemm_fp8_pair_kernel<MXF4> (grouped)")
    out["dgrad"] = _tensor_rec(flops, time_cuda(lambda: gg4.grouped_gemm_fp4_impl(g_row, w_col, g_s_row, w_s_col, lens_t, orow2, out_dtype=torch.bfloat16, group_offs_out=offs), iters),
                               peaks, "fp4", "gemm_fp8_pair_kernel<MXF4> (grouped)")
    out["wgrad"] = _tensor_rec(flops, time_cuda(lambda: gg4.grouped_gemm_fp4_variable_k_impl(g_col, a_col, g_s_col, a_s_col, lcol, ocol, torch.bfloat16), iters),
                               peaks, "fp4", "gemm_fp8_pair_kernel<MXF4> (variable K)")
    return out


def mxfp4_c5_sweep(dev, peaks, tokens_per_expert=(128, 512, 2048, 8192, 16384)):
    """Forward TFLOP/s of the balanced tokens-per-expert sweep of C5."""
    out = {}
    for t in tokens_per_expert:
        rec = grouped_mxfp4_c5(dev, peaks, lens=[t] * C5["G"], iters=6)
        out[str(t)] = {"fwd_tflops": rec["fwd"]["tflops"], "dgrad_tflops": rec["dgrad"]["tflops"], "wgrad_tflops": rec["wgrad"]["tflops"]}
        torch.cuda.empty_cache()
    return out


# ---------------------------------------------------------------------------------------------- rows around the GEMMs
def streaming_records(dev, peaks):
    """Gated activation, RMSNorm and MoE permutation kernels on C4-like tensors; GB/s of algorithmic bytes."""
    from primus_turbo.pytorch.kernels.activation.glu_impl import glu_bwd_with_probs, glu_fwd_with_probs
    from primus_turbo.pytorch.kernels.moe import permutation_impl as pm
    from primus_turbo.pytorch.kernels.normalization import rmsnorm_impl as rn
    out = {}

    def run(name, fns, nbytes, kernel):
        out[name] = _hbm_rec(nbytes, time_cuda_rotating(fns), peaks, kernel)

    rows, inter = 32768, C4["inter"]
    xs = [randn_bf16((rows, 2 * inter), 1.0, 90 + i, dev) for i in range(3)]
    g = randn_bf16((rows, inter), 1.0, 93, dev)
    probs = torch.rand(rows, device=dev, generator=torch.Generator(device=dev).manual_seed(94))
    eo = rows * inter
    run(f"swiglu_fwd_{rows}x{inter}", [lambda x=x: glu_fwd_with_probs(x, probs, None, "silu") for x in xs], 6 * eo + 4 * rows, "glu_fwd_kernel")
    run(f"swiglu_bwd_{rows}x{inter}", [lambda x=x: glu_bwd_with_probs(g, x, probs, None, "silu") for x in xs], 10 * eo + 8 * rows, "glu_bwd_kernel")
    del xs, g
    tokens, hidden = 16384, C4["hidden"]
    hs = [randn_bf16((tokens, hidden), 1.0, 95 + i, dev) for i in range(3)]
    gamma = randn_bf16((hidden,), 1.0, 98, dev)
    e = tokens * hidden
    run(f"rmsnorm_fwd_{tokens}x{hidden}", [lambda x=x: rn.rmsnorm_fwd_impl(x, gamma, 1e-6) for x in hs], 4 * e + 4 * tokens, "rmsnorm_fwd_kernel")
    y, x2, rstd = rn.rmsnorm_fwd_impl(hs[0], gamma, 1e-6)
    run(f"rmsnorm_bwd_{tokens}x{hidden}", [lambda x=x: rn.rmsnorm_bwd_impl(y, x, gamma, rstd) for x in hs], 6 * e, "rmsnorm_bwd_kernel + rmsnorm_dgamma_kernel")
    del y, x2
    # top-8 routing of 16384 tokens over 256 experts (C4): 131072 permuted rows of 7168 bf16
    E, topk = C4["G"], 8
    gen = torch.Generator(device=dev).manual_seed(99)
    scores = torch.rand(tokens, E, device=dev, generator=gen)
    routing = torch.zeros(tokens, E, dtype=torch.bool, device=dev)
    routing.scatter_(1, scores.topk(topk, dim=1).indices, True)
    row_id_map, _ = pm.make_row_id_map(routing, tokens, E)
    n_out = tokens * topk
    run(f"moe_row_id_map_{tokens}x{E}", [lambda: pm.make_row_id_map(routing, tokens, E) for _ in range(2)], tokens * E * (1 + 8) + 4 * tokens, "moe_rank / offs / compact kernels")
    run(f"moe_permute_{tokens}x{hidden}_top{topk}", [lambda x=x: pm.permute_with_mask_map(x, row_id_map, None, None, tokens, E, n_out, hidden) for x in hs],
        2 * e + 2 * n_out * hidden, "moe_permute_kernel")
    perm = pm.permute_with_mask_map(hs[0], row_id_map, None, None, tokens, E, n_out, hidden)[0]
    run(f"moe_unpermute_{tokens}x{hidden}_top{topk}", [lambda: pm.unpermute_with_mask_map(perm, row_id_map, None, None, tokens, E, hidden) for _ in range(2)],
        2 * n_out * hidden + 2 * e, "moe_unpermute_kernel")
    return out


# ---------------------------------------------------------------------------------------------- small cases for profiling
def _small_case(name, args):
    """Runs one kernel a few times on a small input (larger than L2, a few hundred MB on the device): the command line an
    ncu capture of that kernel wraps.  python bench_configs.py <case> [sizes...]"""
    import primus_turbo.pytorch  # noqa: F401  (loads the library)
    from primus_turbo.pytorch.core.low_precision import ScalingGranularity as SG
    from primus_turbo.pytorch.kernels.grouped_gemm import grouped_gemm_fp8_impl as ggi
    from primus_turbo.pytorch.kernels.quantization import quantization_impl as qi
    dev = torch.device("cuda", 0)
    f8, f5 = torch.float8_e4m3fn, torch.float8_e5m2
    if name in ("mx_dual", "mxfp4_dual", "blockwise_dual", "swiglu_mx_dual"):
        M, N = (int(args[0]), int(args[1])) if len(args) >= 2 else (8192, 4096)
        xs = [randn_bf16((M, N * (2 if name == "swiglu_mx_dual" else 1)), 1.0, i, dev) for i in range(3)]
        probs = torch.rand(M, device=dev)
        for i in range(6):
            x = xs[i % 3]
            if name == "mx_dual":
                qi.quantize_mxfp8_impl(x, f8, None, 32, True)
            elif name == "mxfp4_dual":
                qi.quantize_mxfp4_impl(x, torch.float4_e2m1fn_x2, None, 32, True)
            elif name == "blockwise_dual":
                qi.quant_fp8_blockwise_dual_impl(x, f8)
            else:
                qi.glu_quantize_mx_impl(x, probs, None, "silu", f8, fused=True)
    elif name == "blockwise_grouped":   # forward + variable-K wgrad of G equal groups, C4 gate_up widths
        G, per = (int(args[0]), int(args[1])) if len(args) >= 2 else (64, 512)
        N, K = C4["inter2"], C4["hidden"]
        lens = np.full(G, per, dtype=np.int64)
        lens_t, offs = offsets_of(lens, dev)
        x = randn_bf16((G * per, K), 1.0, 1, dev)
        dy = randn_bf16((G * per, N), 1e-3, 2, dev)
        w = randn_bf16((G, N, K), 0.02, 3, dev)
        a_row, a_col, a_s_row, a_s_col, plens, poffs = qi.quant_fp8_blockwise_segment_m_row_col_impl(x, f8, 128, lens_t, offs)
        g_row, g_col, g_s_row, g_s_col, _, _ = qi.quant_fp8_blockwise_segment_m_row_col_impl(dy, f5, 128, lens_t, offs)
        w_q, w_s = qi.quant_fp8_blockwise_for_weight_impl(w, f8)
        for _ in range(2):
            ggi.grouped_gemm_fp8_impl(a_row, w_q, a_s_row, w_s, lens_t, offs, False, True, torch.bfloat16, SG.BLOCKWISE)
            ggi.grouped_gemm_fp8_variable_k_impl(a_col, g_col, a_s_col, g_s_col, plens, poffs, True, False, True, torch.bfloat16, SG.BLOCKWISE)
    elif name == "mx_c3":   # forward and wgrad GEMM of the C3 linear (or of M N K given), one launch each after the quantizers
        from primus_turbo.pytorch.kernels.gemm.gemm_fp8_impl import gemm_fp8_impl
        M, N, K = (int(args[0]), int(args[1]), int(args[2])) if len(args) >= 3 else (C3["M"], C3["N"], C3["K"])
        x = randn_bf16((M, K), 1.0, 71, dev)
        w = randn_bf16((N, K), 0.01, 72, dev)
        dy = randn_bf16((M, N), 1e-3, 73, dev)
        a_row, a_row_s, a_col, a_col_s = qi.quantize_mxfp8_impl(x, f8, None, 32, True)
        b_row, b_row_s, _, _ = qi.quantize_mxfp8_impl(w, f8, None, 32, True)
        _, _, g_col, g_col_s = qi.quantize_mxfp8_impl(dy, f5, None, 32, True)
        del x, w, dy
        for _ in range(2):
            gemm_fp8_impl(a_row, a_row_s, False, b_row, b_row_s, True, torch.bfloat16, False, SG.MX_BLOCKWISE)
            gemm_fp8_impl(g_col, g_col_s, False, a_col, a_col_s, True, torch.bfloat16, False, SG.MX_BLOCKWISE)
    elif name in ("rmsnorm_mx_row", "glu_mx_row"):   # the one-pass forward-only forms
        M, N = (int(args[0]), int(args[1])) if len(args) >= 2 else (8192, 4096)
        xs = [randn_bf16((M, N * (2 if name == "glu_mx_row" else 1)), 1.0, i, dev) for i in range(3)]
        gamma = randn_bf16((N,), 1.0, 7, dev)
        probs = torch.rand(M, device=dev)
        for i in range(6):
            if name == "rmsnorm_mx_row":
                qi.rmsnorm_quantize_mx_row_impl(xs[i % 3], gamma, 1e-6, False, f8, fused=True)
            else:
                qi.glu_quantize_mx_row_impl(xs[i % 3], probs, None, "silu", f8, fused=True)
    elif name in ("rowwise_other_axis", "rmsnorm_bwd", "rmsnorm_mx_dual"):
        from primus_turbo.pytorch.kernels.normalization import rmsnorm_impl as ri
        M, N = (int(args[0]), int(args[1])) if len(args) >= 2 else (8192, 4096)
        xs = [randn_bf16((M, N), 1.0, i, dev) for i in range(3)]
        gamma = randn_bf16((N,), 1.0, 7, dev)
        dy = randn_bf16((M, N), 1e-2, 8, dev)
        rstd = ri.rmsnorm_stats_impl(xs[0], 1e-6)
        for i in range(6):
            x = xs[i % 3]
            if name == "rowwise_other_axis":
                qi.quantize_fp8_rowwise_impl(x, f8, -2)
            elif name == "rmsnorm_bwd":
                ri.rmsnorm_bwd_impl(dy, x, gamma, rstd)
            else:
                qi.rmsnorm_quantize_mx_impl(x, gamma, 1e-6, False, f8, fused=True)
    else:
        raise SystemExit(f"unknown case {name!r}: mx_dual, mxfp4_dual, blockwise_dual, swiglu_mx_dual, rowwise_other_axis, "
                         "rmsnorm_bwd, rmsnorm_mx_dual, rmsnorm_mx_row, glu_mx_row [M N]; blockwise_grouped [G rows]; mx_c3 [M N K]")
    torch.cuda.synchronize()
    print("ok", name, *args)


if __name__ == "__main__":
    import os
    import sys
    sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "primus-turbo_b200"))
    _small_case(sys.argv[1] if len(sys.argv) > 1 else "", sys.argv[2:])
