"""Benchmark of the low-precision GEMM hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

One "pass" is the forward of gemm_fp8(a, w, trans_b=True, config=MX_BLOCKWISE) exactly as the reference's operator
does it (primus_turbo/pytorch/ops/gemm_fp8.py:558-654): dual (row + transposed col) MX quantization of the activation
and of the weight, then the MXFP8 GEMM.  Default workload: the Llama-3-8B MLP shape M=8192, K=4096, N=14336 that the
north-star throughput target is quoted on.  One "step" is R back-to-back passes (`config.inner_repeats`), R chosen
from the warm-up so that the K timed steps last about 1.5 s: the GPU then runs at the clock it sustains under its
power limit, not at the boost clock of a 10 ms burst.

Rank 0 prints one JSON line.  `value` is 2*M*N*K*R / step time summed over ranks (TFLOPS, inputs resident in HBM);
`e2e` is the same metric through the public operator with pinned host buffers, host<->device copies inside the timed
region; `roofline` describes the GEMM kernel (tensor bound); `cpu_baseline` is the torch-CPU port of the same pass.
`sub` holds the other benchmark configurations (bench_configs.py): quantizer GB/s, dense backward, the MXFP8 70B
FFN shape, the blockwise MoE grouped GEMMs, the MXFP4 grouped GEMMs (and their tokens-per-expert sweep) and the
streaming kernels around them (gated activation, RMSNorm, MoE permutation), each with its own roofline record; with
N > 1 instead the expert-sharded and N-sharded runs through primus_turbo.pytorch.dist.partitioner.
"""
import argparse
import json
import os
import statistics
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
for p in (ROOT, os.path.join(ROOT, "primus-turbo_b200")):
    if p not in sys.path:
        sys.path.insert(0, p)

import torch  # noqa: E402

WORKLOADS = {
    # name: (M, N, K, seed)  -- Llama-3 MLP / FFN shapes of the benchmark configurations; activations ~N(0,1) with 0.1% x50 outliers, weights ~N(0,0.02)
    "mxfp8_linear_fwd_llama3_8b_mlp": (8192, 14336, 4096, 1),
    "mxfp8_linear_fwd_llama3_70b_ffn": (16384, 28672, 8192, 2),
}
DEFAULT_WORKLOAD = "mxfp8_linear_fwd_llama3_8b_mlp"
# DRAM bytes (read + write) of one GEMM launch from the ncu capture summarised in
# profiles/gemm_mxfp8_pair_8192x14336x4096.md; null until that capture exists for the workload.
GEMM_DRAM_TRAFFIC = {"mxfp8_linear_fwd_llama3_8b_mlp": 334.6e6}
TARGET_TIMED_SECONDS = 1.5


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return {"hbm_gbs": d["hbm_gbs"], "bf16_burst": d["bf16_tflops"], "bf16_sustained": d["bf16_tflops_sustained"],
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_burst": 1590.0, "bf16_sustained": 1400.0, "source": "fallback"}


def make_inputs(M, N, K, seed, device):
    """Seeded synthetic inputs generated on the CPU, returned as pinned host tensors."""
    g = torch.Generator().manual_seed(seed)
    a = torch.randn(M, K, generator=g)
    a = torch.where(torch.rand(M, K, generator=g) < 0.001, a * 50, a).to(torch.bfloat16)
    w = (0.02 * torch.randn(N, K, generator=g)).to(torch.bfloat16)
    if device != "cpu":
        a, w = a.pin_memory(), w.pin_memory()
    return a, w


class ClockSampler:
    """Reads (never sets) SM clock and throttle reasons through NVML from a thread while the timed region runs."""

    def __init__(self, index, period_s=0.002):
        self.index, self.period, self.samples, self.reasons, self.max_mhz = index, period_s, [], set(), None
        self._stop, self._thread, self._err = None, None, None

    def start(self):
        import threading
        try:
            import pynvml
            pynvml.nvmlInit()
            # honour CUDA_VISIBLE_DEVICES: NVML indexes physical devices
            vis = os.environ.get("CUDA_VISIBLE_DEVICES")
            phys = self.index
            if vis:
                ids = [v.strip() for v in vis.split(",") if v.strip()]
                if self.index < len(ids) and ids[self.index].isdigit():
                    phys = int(ids[self.index])
            h = pynvml.nvmlDeviceGetHandleByIndex(phys)
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(h, pynvml.NVML_CLOCK_SM))
        except Exception as e:  # noqa: BLE001
            self._err = repr(e)
            return
        names = {"hw_slowdown": pynvml.nvmlClocksEventReasonHwSlowdown if hasattr(pynvml, "nvmlClocksEventReasonHwSlowdown") else 0x8,
                 "hw_thermal_slowdown": 0x40, "sw_thermal_slowdown": 0x20, "sw_power_cap": 0x4}
        self._stop = threading.Event()

        def loop():
            while not self._stop.is_set():
                try:
                    self.samples.append(float(pynvml.nvmlDeviceGetClockInfo(h, pynvml.NVML_CLOCK_SM)))
                    try:
                        mask = pynvml.nvmlDeviceGetCurrentClocksEventReasons(h)
                    except Exception:  # noqa: BLE001
                        mask = pynvml.nvmlDeviceGetCurrentClocksThrottleReasons(h)
                    for n, bit in names.items():
                        if mask & bit:
                            self.reasons.add(n)
                except Exception as e:  # noqa: BLE001
                    self._err = repr(e)
                    return
                time.sleep(self.period)

        self._thread = threading.Thread(target=loop, daemon=True)
        self._thread.start()

    def stop(self):
        if self._thread is not None:
            self._stop.set()
            self._thread.join(timeout=2)
        out = {"sm_mhz": statistics.median(self.samples) if self.samples else None, "sm_max_mhz": self.max_mhz,
               "reasons": sorted(self.reasons), "samples": len(self.samples)}
        if self._err:
            out["error"] = self._err
        return out


def cpu_baseline(M, N, K, seed, sample_rows=1024):
    """The same pass on the host cores (torch-CPU port of the path).  The weight half (dual quantization of the full
    weight, done once per pass whatever M is) is timed in full; the activation half (dual quantization of the
    activation and the GEMM, both linear in the rows) is timed on `sample_rows` of the M rows and scaled by
    M / sample_rows.  value = 2*M*N*K / (t_weight + t_activation * M / sample_rows)."""
    from oracle import torch_port as tp
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    a, w = make_inputs(sample_rows, N, K, seed, "cpu")
    tp.mx_linear_forward(a[:64], w[:128])  # warm the thread pool
    t0 = time.perf_counter()
    w_deq = tp.mx_weight_prepare(w)
    t1 = time.perf_counter()
    tp.mx_activation_forward(a, w_deq)
    t2 = time.perf_counter()
    t_w, t_a = t1 - t0, t2 - t1
    full = t_w + t_a * (M / sample_rows)
    return {"value": 2.0 * M * N * K / full / 1e12, "unit": "TFLOPS", "cores": cores, "kind": "port",
            "sample": f"weight half (dual 2-D MX quantization of [{N}x{K}]) in full: {t_w:.2f} s; activation half (dual MX "
                      f"quantization + fp32 GEMM) on {sample_rows} of {M} rows: {t_a:.2f} s, scaled x{M // sample_rows}; "
                      f"full pass = {full:.2f} s",
            "seconds": t_w + t_a, "seconds_full_pass": full}


def run_reference(args, M, N, K, seed, workload):
    """--impl reference: the path's CPU implementation on the host cores.  The reference's own kernels are
    HIP / Triton / FlyDSL for AMD GPUs and cannot run here; its CPU-runnable form is the torch port."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    sample_rows = 1024
    fulls, secs = [], []
    for i in range(args.warmup + args.steps):
        r = cpu_baseline(M, N, K, seed, sample_rows)
        if i >= args.warmup:
            fulls.append(r["seconds_full_pass"])
            secs.append(r["seconds"])
    ms = 1e3 * sum(secs) / len(secs)
    value = 2.0 * M * N * K / (sum(fulls) / len(fulls)) / 1e12
    base = dict(r)
    base["value"] = value
    base.pop("seconds")
    base.pop("seconds_full_pass")
    print(json.dumps({
        "impl": "reference", "metric": "MXFP8 linear forward (dual quantize x2 + GEMM) throughput", "value": value,
        "unit": "TFLOPS", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "fp8_e4m3 (fp32 accumulate)",
        "data": "synthetic", "config": {"workload": workload, "M": M, "N": N, "K": K, "granularity": "MX_BLOCKWISE",
                                        "format": "E4M3", "out_dtype": "bf16"},
        "cpu_baseline": base,
        "e2e": {"value": value, "unit": "TFLOPS", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}))


def _sub_records(args, dev, peaks, world, rank):
    """The other benchmark configurations; every entry is self-contained and a failing one does not sink the line."""
    import bench_configs as bc
    sub = {}

    def attempt(name, fn):
        sampler = ClockSampler(dev.index or 0, period_s=0.005)
        if rank == 0:
            sampler.start()
        try:
            sub[name] = fn()
        except Exception as exc:  # noqa: BLE001
            sub[name] = {"error": repr(exc)[:300]}
        if rank == 0 and isinstance(sub[name], dict):
            c = sampler.stop()
            sub[name]["clocks"] = {"sm_mhz": c["sm_mhz"], "reasons": c["reasons"], "samples": c["samples"]}
        torch.cuda.empty_cache()

    if world == 1:
        # the bandwidth-bound records first, before the GEMM records have pushed the GPU into its power cap
        attempt("quantize", lambda: bc.quantize_records(dev, peaks))
        attempt("streaming_f2_f4", lambda: bc.streaming_records(dev, peaks))
        attempt("dense_bwd_c2", lambda: bc.dense_bwd_c2(dev, peaks))
        attempt("mx_c3", lambda: bc.mx_c3(dev, peaks))
        attempt("grouped_blockwise_c4", lambda: bc.grouped_blockwise_c4(dev, peaks))
        attempt("grouped_mxfp4_c5", lambda: bc.grouped_mxfp4_c5(dev, peaks))
        attempt("grouped_mxfp4_c5_sweep", lambda: bc.mxfp4_c5_sweep(dev, peaks))
    else:
        import bench_sharded as bs
        attempt("expert_sharded_c4", lambda: bs.expert_sharded_c4(dev, peaks, world, rank))
        attempt("expert_sharded_c4_row_balanced", lambda: bs.expert_sharded_c4(dev, peaks, world, rank, balance="rows"))
        attempt("n_sharded_c3", lambda: bs.n_sharded_c3(dev, peaks, world, rank))
    return sub


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default=DEFAULT_WORKLOAD, choices=sorted(WORKLOADS))
    ap.add_argument("--granularity", default="mx", choices=["mx", "blockwise", "tensorwise", "rowwise", "mxfp4", "bf16"],
                    help="scaling recipe of the linear forward; the headline metric is 'mx' (the others print the same "
                         "line for their own kernels and skip the CPU leg and the other configurations)")
    ap.add_argument("--inner-repeats", type=int, default=0, help="passes per step; 0 = sized from the warm-up so that the "
                                                                 "timed steps last about 1.5 s")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer leg (used when profiling)")
    ap.add_argument("--no-sub", action="store_true", help="skip the other configurations (used when profiling)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    M, N, K, seed = WORKLOADS[args.workload]

    if args.impl == "reference":
        if args.granularity != "mx":
            print(json.dumps({"impl": "reference", "unavailable": "the CPU port covers the MX_BLOCKWISE headline workload only"}))
            return
        run_reference(args, M, N, K, seed, args.workload)
        return

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)

    import primus_turbo.pytorch as turbo
    from primus_turbo.pytorch.core.low_precision import (Float8QuantConfig, Format, ScaleDtype, ScalingGranularity,
                                                         ScalingRecipe)
    from primus_turbo.pytorch.kernels import _native as nv
    from primus_turbo.pytorch.kernels.gemm.gemm_fp8_impl import gemm_fp8_impl
    from primus_turbo.pytorch.kernels.gemm.gemm_fp4_impl import gemm_fp4_impl
    from primus_turbo.pytorch.kernels.quantization import quantization_impl as qi
    from primus_turbo.pytorch.kernels.quantization.quantization_impl import quantize_mxfp8_impl

    if args.granularity == "bf16":
        cfg, public_op = None, (lambda x, y, trans_b, out_dtype, config: turbo.ops.gemm(x, y, trans_b=trans_b, out_dtype=out_dtype))
    elif args.granularity == "mxfp4":
        from primus_turbo.pytorch.core.low_precision import Float4QuantConfig
        cfg, public_op = Float4QuantConfig(), turbo.ops.gemm_fp4
    elif args.granularity == "mx":
        cfg = Float8QuantConfig(format=Format.E4M3, granularity=ScalingGranularity.MX_BLOCKWISE, scale_dtype=ScaleDtype.E8M0,
                                block_size=32)
        public_op = turbo.ops.gemm_fp8
    else:
        gran = {"blockwise": ScalingGranularity.BLOCKWISE, "tensorwise": ScalingGranularity.TENSORWISE,
                "rowwise": ScalingGranularity.ROWWISE}[args.granularity]
        cfg = Float8QuantConfig(format=Format.E4M3, granularity=gran, block_size=128 if args.granularity == "blockwise" else None)
        public_op = turbo.ops.gemm_fp8
    # The other configurations run first, each kernel timed alone in short loops on a GPU that has not yet been driven
    # into its power limit (their denominators are the burst figures); the long headline region follows.
    peaks = measured_peaks()
    sub = None
    if args.granularity == "mx" and not args.no_sub and args.workload == DEFAULT_WORKLOAD:
        sub = _sub_records(args, dev, peaks, world, rank)
        nv.check_status(dev)

    # weak scaling: every rank owns one N-shard of a layer that is `world` times as wide (its own weight shard),
    # the activation is replicated; no collective on the data path (outputs stay column-sharded).
    a_host, w_host = make_inputs(M, N, K, seed + 1000 * rank, "cuda")
    a = a_host.to(dev, non_blocking=True)
    w = w_host.to(dev, non_blocking=True)
    torch.cuda.synchronize()
    f8 = torch.float8_e4m3fn
    plain, two_d = ScalingRecipe(), ScalingRecipe(use_2d_block=True)
    gemm_events = []

    G = ScalingGranularity
    # per recipe: (quantize both operands the way the reference's forward does, GEMM on the quantized operands,
    #              launches of this library per pass, name of the dominant kernel)
    if args.granularity == "mx":
        quant = lambda: (quantize_mxfp8_impl(a, f8, None, 32, True, plain, plain)[:2],
                         quantize_mxfp8_impl(w, f8, None, 32, True, two_d, two_d)[:2])
        gemm = lambda qa, qw: gemm_fp8_impl(qa[0], qa[1], False, qw[0], qw[1], True, torch.bfloat16, False, G.MX_BLOCKWISE)
        launches, kernel_name = 4, "gemm_fp8_pair_kernel<MX>"  # 2 dual quantize, 1 scale re-tile, 1 GEMM
    elif args.granularity == "mxfp4":
        fp4 = torch.float4_e2m1fn_x2
        quant = lambda: (qi.quantize_mxfp4_impl(a, fp4, None, 32, True, plain, plain)[:2],
                         qi.quantize_mxfp4_impl(w, fp4, None, 32, True, two_d, two_d)[:2])
        gemm = lambda qa, qw: gemm_fp4_impl(qa[0], qa[1], False, qw[0], qw[1], True, torch.bfloat16, False, G.MX_BLOCKWISE)
        launches, kernel_name = 4, "gemm_fp8_pair_kernel<MXF4>"
    elif args.granularity == "bf16":
        from primus_turbo.pytorch.kernels.gemm.gemm_impl import gemm_impl
        quant = lambda: (a, w)   # nothing to quantize: the comparison line of the low-precision recipes
        gemm = lambda qa, qw: gemm_impl(qa, False, qw, True, torch.bfloat16, False)
        launches, kernel_name = 1, "gemm_fp8_pair_kernel<HP>"
    elif args.granularity == "blockwise":
        quant = lambda: (qi.quant_fp8_blockwise_impl(a, f8, 1), qi.quant_fp8_blockwise_for_weight_impl(w, f8))
        gemm = lambda qa, qw: gemm_fp8_impl(qa[0], qa[1], False, qw[0], qw[1], True, torch.bfloat16, False, G.BLOCKWISE)
        launches, kernel_name = 3, "gemm_fp8_blockwise_kernel<SB_TILE>"
    else:
        gran = G.TENSORWISE if args.granularity == "tensorwise" else G.ROWWISE
        if gran == G.TENSORWISE:
            quant = lambda: (qi.quantize_fp8_tensorwise_impl(a, f8), qi.quantize_fp8_tensorwise_impl(w, f8))
        else:
            quant = lambda: (qi.quantize_fp8_rowwise_impl(a, f8, -1), qi.quantize_fp8_rowwise_impl(w, f8, -1))
        gemm = lambda qa, qw: gemm_fp8_impl(qa[0], qa[1], False, qw[0], qw[1], True, torch.bfloat16, False, gran)
        launches, kernel_name = (5 if gran == G.TENSORWISE else 3), f"gemm_fp8_kernel<{args.granularity.upper()}>"

    def one_pass(record=False):
        qa, qw = quant()
        if record:
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
        out = gemm(qa, qw)
        if record:
            e1.record()
            gemm_events.append((e0, e1))
        return out

    def barrier():
        if world > 1:
            import torch.distributed as dist
            dist.barrier()
        torch.cuda.synchronize()

    # warm-up; the last warm-up passes also size the step
    for _ in range(args.warmup):
        one_pass()
    barrier()
    repeats = args.inner_repeats
    if repeats <= 0:
        p0, p1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        p0.record()
        for _ in range(10):
            one_pass()
        p1.record()
        torch.cuda.synchronize()
        pass_ms = p0.elapsed_time(p1) / 10
        rep = torch.tensor([max(1, min(2000, round(TARGET_TIMED_SECONDS * 1e3 / (args.steps * pass_ms))))], dtype=torch.int64, device=dev)
        if world > 1:
            import torch.distributed as dist
            dist.all_reduce(rep, op=dist.ReduceOp.MAX)
        repeats = int(rep.item())

    def step():
        for r in range(repeats):
            out = one_pass(record=(r == 0))   # one GEMM-only event pair per step keeps the event count bounded
        return out

    for _ in range(2):
        step()
    gemm_events.clear()
    barrier()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    t_begin, t_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    t_begin.record()
    for _ in range(args.steps):
        step()
    t_end.record()
    barrier()
    clocks = sampler.stop() if rank == 0 else None
    nv.check_status(dev)
    ms_total = t_begin.elapsed_time(t_end)
    gemm_ms = sum(e0.elapsed_time(e1) for e0, e1 in gemm_events) / len(gemm_events)

    # N > 1: the same passes with the output columns of all ranks gathered on every rank (one NCCL all_gather per
    # pass, the collective of a column-parallel linear with gather_output); reported beside `value`, not in it.
    gather_ms, gather_error, n_gather = 0.0, None, 0
    if world > 1:
        try:
            import torch.distributed as dist
            # rank-major blocks [world][M, N], two buffers: the gather of pass i runs on its own stream under pass i + 1
            recv = [torch.empty((world * M, N), dtype=torch.bfloat16, device=dev) for _ in range(2)]
            comm = torch.cuda.Stream()
            main_stream = torch.cuda.current_stream()

            def gather_step(i):
                out = one_pass()
                done = torch.cuda.Event()
                done.record(main_stream)
                with torch.cuda.stream(comm):
                    comm.wait_event(done)
                    dist.all_gather_into_tensor(recv[i % 2], out)
                    out.record_stream(comm)

            for i in range(3):
                gather_step(i)
            main_stream.wait_stream(comm)
            barrier()
            n_gather = max(20, min(200, args.steps * repeats // 8))
            g_begin, g_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            g_begin.record()
            for i in range(n_gather):
                gather_step(i)
            main_stream.wait_stream(comm)   # the last gather is inside the timed region
            g_end.record()
            barrier()
            gather_ms = g_begin.elapsed_time(g_end)
            del recv
        except Exception as exc:  # the line without the gather is still valid
            gather_ms, gather_error = float('nan'), repr(exc)[:200]

    # End to end through the public operator, host buffers in and out.  Every pass uploads its inputs from pinned host
    # memory and downloads its result; uploads, compute and downloads run on three streams over two sets of device
    # buffers, so pass i + 1's upload overlaps pass i's download (PCIe is full duplex) — all inside the timed region.
    out_host = [torch.empty((M, N), dtype=torch.bfloat16).pin_memory() for _ in range(2)]
    a_dev = [torch.empty_like(a) for _ in range(2)]
    w_dev = [torch.empty_like(w) for _ in range(2)]
    main = torch.cuda.current_stream()
    up, down = torch.cuda.Stream(), torch.cuda.Stream()
    uploaded = [torch.cuda.Event() for _ in range(2)]
    computed = [torch.cuda.Event() for _ in range(2)]
    downloaded = [torch.cuda.Event() for _ in range(2)]
    results = [None, None]

    def e2e_step(i):
        s = i & 1
        with torch.cuda.stream(up):
            up.wait_event(computed[s])        # the compute that read this input set two passes ago is done
            a_dev[s].copy_(a_host, non_blocking=True)
            w_dev[s].copy_(w_host, non_blocking=True)
            uploaded[s].record(up)
        main.wait_event(uploaded[s])
        main.wait_event(downloaded[s])       # the result buffer of two passes ago has left the device
        results[s] = public_op(a_dev[s], w_dev[s], trans_b=True, out_dtype=torch.bfloat16, config=cfg)
        computed[s].record(main)
        with torch.cuda.stream(down):
            down.wait_event(computed[s])
            out_host[s].copy_(results[s], non_blocking=True)
            downloaded[s].record(down)

    with torch.no_grad():
        for i in range(0 if args.no_e2e else 4):
            e2e_step(i)
        barrier()
        e_begin, e_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        n_e2e = 0 if args.no_e2e else max(4, min(args.steps, 12))
        e_begin.record()
        for i in range(n_e2e):
            e2e_step(i)
        main.wait_stream(down)               # the last downloads are part of the measurement
        main.wait_stream(up)
        e_end.record()
        barrier()
    e2e_ms = e_begin.elapsed_time(e_end) / n_e2e if n_e2e else float('nan')
    del a_dev, w_dev, results
    torch.cuda.empty_cache()

    t = torch.tensor([ms_total, gemm_ms, e2e_ms, gather_ms], dtype=torch.float64, device=dev)
    if world > 1:
        import torch.distributed as dist
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_total, gemm_ms, e2e_ms, gather_ms = (float(v) for v in t.tolist())
    ms_per_step = ms_total / args.steps
    ms_per_pass = ms_per_step / repeats
    flops = 2.0 * M * N * K

    if rank != 0:
        if world > 1:
            import torch.distributed as dist
            dist.destroy_process_group()
        return
    # Denominator by regime: a timed region of a second or more runs under the power limit (the sustained figure); a
    # shorter one at the boost clock (the burst figure).  FP8 = 2 x, FP4 = 4 x the measured bf16 GEMM.
    mult = {"mxfp4": 4.0, "bf16": 1.0}.get(args.granularity, 2.0)
    sustained_regime = ms_total >= 1000.0
    peak_burst, peak_sustained = mult * peaks["bf16_burst"], mult * peaks["bf16_sustained"]
    tensor_peak = peak_sustained if sustained_regime else peak_burst
    achieved = flops / (gemm_ms / 1e3) / 1e12
    if clocks and clocks.get("sm_mhz"):
        clocks["pass_ms_x_sm_mhz"] = ms_per_pass * clocks["sm_mhz"]
    recipe = {"mx": ("MXFP8 linear forward (dual quantize x2 + GEMM) throughput", "MX_BLOCKWISE", "E4M3", "fp8_e4m3 (fp32 accumulate)"),
              "mxfp4": ("MXFP4 linear forward (dual quantize x2 + GEMM) throughput", "MX_BLOCKWISE", "E2M1_X2", "fp4_e2m1 (fp32 accumulate)"),
              "blockwise": ("FP8 blockwise linear forward (quantize x2 + GEMM) throughput", "BLOCKWISE", "E4M3", "fp8_e4m3 (fp32 accumulate)"),
              "tensorwise": ("FP8 tensorwise linear forward (quantize x2 + GEMM) throughput", "TENSORWISE", "E4M3", "fp8_e4m3 (fp32 accumulate)"),
              "rowwise": ("FP8 rowwise linear forward (quantize x2 + GEMM) throughput", "ROWWISE", "E4M3", "fp8_e4m3 (fp32 accumulate)"),
              "bf16": ("BF16 linear forward (GEMM) throughput", "NONE", "BF16", "bf16 (fp32 accumulate)")}[args.granularity]
    quant_ms = ms_per_pass - gemm_ms
    result = {
        "metric": recipe[0], "value": world * flops / (ms_per_pass / 1e3) / 1e12,
        "unit": "TFLOPS", "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": recipe[3],
        "data": "synthetic",
        "config": {"workload": args.workload, "M": M, "N": N, "K": K, "granularity": recipe[1], "format": recipe[2],
                   "out_dtype": "bf16", "inner_repeats": repeats, "ms_per_pass": ms_per_pass,
                   "per_gpu_shard": f"activation replicated, weight shard [{N}x{K}] per GPU",
                   "l2": "inputs 184 MB per pass exceed the 126 MB L2; no flush between iterations"},
        "roofline": {"bound": "tensor", "achieved": achieved, "peak": tensor_peak, "unit": "TFLOP/s", "frac": achieved / tensor_peak,
                     "traffic": GEMM_DRAM_TRAFFIC.get(args.workload) if args.granularity == "mx" else None, "kernel": kernel_name,
                     "regime": "sustained (timed region >= 1 s)" if sustained_regime else "burst (timed region < 1 s)",
                     "peak_source": f"{mult:g} x bf16_tflops{'_sustained' if sustained_regime else ''} of {peaks['source']} MEASURED_PEAKS.json",
                     "frac_of_burst_peak": achieved / peak_burst, "frac_of_sustained_peak": achieved / peak_sustained,
                     "gemm_ms_per_launch": gemm_ms,
                     "frac_of_nominal": achieved / {"mxfp4": 9000.0, "bf16": 2250.0}.get(args.granularity, 4500.0)},
        "clocks": clocks,
        "e2e": {"value": None if args.no_e2e else world * flops / (e2e_ms / 1e3) / 1e12, "unit": "TFLOPS",
                "h2d_bytes_per_step": a_host.numel() * 2 + w_host.numel() * 2, "d2h_bytes_per_step": out_host[0].numel() * 2,
                "ms_per_step": None if args.no_e2e else e2e_ms, "note": "one pass per e2e step"},
        "gpu_launches": launches * args.steps * repeats,
    }
    if args.granularity in ("mx", "mxfp4"):
        e, ew = M * K, N * K
        per = (0.5 if args.granularity == "mxfp4" else 1.0)
        qbytes = 2 * (e + ew) + 2 * (per + 1 / 32) * (e + ew)
        result["quantize_in_pass"] = {"ms": quant_ms, "bytes": qbytes, "gbs": qbytes / (quant_ms / 1e3) / 1e9,
                                      "frac": qbytes / (quant_ms / 1e3) / 1e9 / peaks["hbm_gbs"],
                                      "what": "pass time minus the GEMM's events: two dual quantizers (+ launch gaps)"}
    if world > 1 and gather_error is not None:
        result["with_output_gather"] = {"value": None, "error": gather_error}
    elif world > 1:
        g_ms = gather_ms / n_gather
        result["with_output_gather"] = {"value": world * flops / (g_ms / 1e3) / 1e12, "unit": "TFLOPS", "ms_per_pass": g_ms,
                                        "collective": f"NCCL all_gather of the [{M}x{N}] bf16 output shard into rank-major blocks, {world} ranks, on a second stream under the next pass",
                                        "gathered_bytes_per_rank": (world - 1) * M * N * 2}
    if sub is not None:
        result["sub"] = sub
    if world == 1 and not args.no_cpu_baseline and args.granularity == "mx":
        cb = cpu_baseline(M, N, K, seed)
        cb.pop("seconds")
        cb.pop("seconds_full_pass")
        result["cpu_baseline"] = cb
    print(json.dumps(result))
    if world > 1:
        import torch.distributed as dist
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
