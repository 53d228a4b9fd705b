"""Sharded measurements of `bench.py --gpus N` (N > 1), through primus_turbo.pytorch.dist.partitioner.

* expert_sharded_c4 — the 256 experts of the blockwise-FP8 MoE configuration split N ways (32 per GPU at N = 8),
  each rank holding its experts' weights and the rows routed to them: total work is fixed ("strong"), the step time
  is the slowest rank's, so the Zipf load imbalance is part of the number.
* n_sharded_c3 — the 16384 x 28672 x 8192 MXFP8 linear split along its output columns.

Times are CUDA events per rank, reduced with MAX over ranks.  Each record gives the figure without the output
gather (outputs stay with their owner, as in an expert-parallel or column-parallel layer) and with it; the gather's
own roofline is the NVLink receive rate of one GPU (770 GB/s measured peer copy).
"""
import torch
import torch.distributed as dist

import bench_configs as bc

NVLINK_GBS = 770.0


def _max_over_ranks(values, dev):
    t = torch.tensor(values, dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return [float(v) for v in t.tolist()]


def _gather_ints(value, world, dev):
    t = torch.zeros(world, dtype=torch.int64, device=dev)
    t[dist.get_rank()] = int(value)
    dist.all_reduce(t, op=dist.ReduceOp.SUM)
    return [int(v) for v in t.tolist()]


def _sum_over_ranks(values, dev):
    t = torch.tensor(values, dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.SUM)
    return [float(v) for v in t.tolist()]


def expert_sharded_c4(dev, peaks, world, rank, projection="gate_up", balance="experts"):
    """balance="experts": 256 / N consecutive experts per rank (the Zipf skew then decides the slowest rank);
    balance="rows": the packed rows split evenly, popular experts shared between neighbouring ranks."""
    import numpy as np
    from primus_turbo.pytorch.core.low_precision import Float8QuantConfig, Format, ScalingGranularity
    from primus_turbo.pytorch.dist.partitioner import ExpertShardedGroupedLinear, expert_shard, row_balanced_expert_shard
    cfg = Float8QuantConfig(format=Format.E4M3, granularity=ScalingGranularity.BLOCKWISE, block_size=128)
    lens_all = bc.zipf_group_lens(bc.C4["G"], bc.C4["rows"], seed=bc.C4["seed"])
    if balance == "rows":
        g_lo, g_hi, lens = row_balanced_expert_shard([int(v) for v in lens_all], world, rank)
        lens = np.asarray(lens, dtype=np.int64)
    else:
        g_lo, g_hi = expert_shard(bc.C4["G"], world, rank)
        lens = lens_all[g_lo:g_hi]
    N, K = (bc.C4["inter2"], bc.C4["hidden"]) if projection == "gate_up" else (bc.C4["hidden"], bc.C4["inter"])
    rows = int(lens.sum())
    lens_t, _ = bc.offsets_of(lens, dev)
    w = bc.randn_bf16((g_hi - g_lo, N, K), 0.02, 83 + g_lo, dev)
    x = bc.randn_bf16((max(rows, 1), K), 1.0, 81 + g_lo, dev)[:rows]
    ex = ExpertShardedGroupedLinear(bc.C4["G"], w, config=cfg, cache_quantized_weight=True, experts=(g_lo, g_hi))
    rows_all = _gather_ints(rows, world, dev)
    with torch.no_grad():
        fwd_ms = bc.time_cuda(lambda: ex.forward(x, lens_t), iters=8)
        dist.barrier()
        gat_ms = bc.time_cuda(lambda: ex.gather_rows(ex.forward(x, lens_t), rows_all), iters=6)
    del ex, w, x
    torch.cuda.empty_cache()
    # kernel-only forward / dgrad / wgrad of this rank's experts (same layouts, quantized operands prepared outside)
    k = bc.grouped_blockwise_c4(dev, peaks, g_lo, g_hi, projections=(projection,), iters=6, lens=lens)[projection]
    ms = _max_over_ranks([fwd_ms, gat_ms, k["fwd"]["ms"], k["dgrad"]["ms"], k["wgrad"]["ms"]], dev)
    rows_max = _max_over_ranks([float(rows)], dev)[0]
    flops = 2.0 * bc.C4["rows"] * N * K
    tf = lambda m: flops / (m / 1e3) / 1e12
    recv_bytes = (bc.C4["rows"] - rows) * N * 2
    return {"scaling": "strong", "projection": projection, "balance": balance, "experts_on_rank0": g_hi - g_lo, "rows_rank0": rows,
            "load_imbalance_max_over_mean": rows_max / (bc.C4["rows"] / world),
            "operator_fwd": {"ms_max_rank": ms[0], "tflops_total": tf(ms[0]),
                             "what": "segment-M quantize of the local rows + grouped GEMM on cached quantized experts"},
            "operator_fwd_with_gather": {"ms_max_rank": ms[1], "tflops_total": tf(ms[1]),
                                         "gather": "padded all_gather of every rank's output rows (NCCL)",
                                         "received_bytes_rank0": recv_bytes,
                                         "nvlink_floor_ms": recv_bytes / NVLINK_GBS / 1e6},
            "gemm_fwd": {"ms_max_rank": ms[2], "tflops_total": tf(ms[2])},
            "gemm_dgrad": {"ms_max_rank": ms[3], "tflops_total": tf(ms[3])},
            "gemm_wgrad": {"ms_max_rank": ms[4], "tflops_total": tf(ms[4])}}


def n_sharded_c3(dev, peaks, world, rank):
    from primus_turbo.pytorch.core.low_precision import Float8QuantConfig, Format, ScaleDtype, ScalingGranularity
    from primus_turbo.pytorch.dist.partitioner import ColumnShardedLinear, column_shard
    cfg = Float8QuantConfig(format=Format.E4M3, granularity=ScalingGranularity.MX_BLOCKWISE, scale_dtype=ScaleDtype.E8M0,
                            block_size=32)
    M, K, N = bc.C3["M"], bc.C3["K"], bc.C3["N"]
    n_lo, n_hi = column_shard(N, world, rank)
    w = bc.randn_bf16((N, K), 0.01, 72, dev)[n_lo:n_hi].contiguous()
    x = bc.randn_bf16((M, K), 1.0, 71, dev)
    lin = ColumnShardedLinear(N, w, config=cfg)
    equal = len({column_shard(N, world, r)[1] - column_shard(N, world, r)[0] for r in range(world)}) == 1
    with torch.no_grad():
        fwd_ms = bc.time_cuda(lambda: lin.forward(x), iters=8)
        dist.barrier()
        into_ms = 0.0
        if equal:
            buf = lin.gather_buffer(M, torch.bfloat16, dev)
            into_ms = bc.time_cuda(lambda: lin.forward_into(x, buf), iters=8)
            dist.barrier()
            gat_ms = bc.time_cuda(lambda: lin.gather_in_place((lin.forward_into(x, buf), buf)[1]), iters=6)
            del buf
        else:
            gat_ms = bc.time_cuda(lambda: lin.gather(lin.forward(x)), iters=6)
    del lin, w, x
    torch.cuda.empty_cache()
    k = bc.mx_c3(dev, peaks, n_lo, n_hi)
    ms = _max_over_ranks([fwd_ms, gat_ms, k["fwd"]["ms"], k["wgrad"]["ms"], into_ms], dev)
    flops = 2.0 * M * N * K
    tf = lambda m: flops / (m / 1e3) / 1e12
    recv_bytes = M * (N - (n_hi - n_lo)) * 2
    return {"scaling": "strong", "columns_per_rank": n_hi - n_lo,
            "operator_fwd": {"ms_max_rank": ms[0], "tflops_total": tf(ms[0]),
                             "what": "dual MX quantize of the replicated activation and of the weight shard + GEMM"},
            "inference_fwd_into_gather_buffer": {"ms_max_rank": ms[4], "tflops_total": tf(ms[4]) if ms[4] else None,
                                                 "what": "no-grad forward: row-wise MX quantize only, GEMM writes its block of the gather buffer"},
            "inference_fwd_with_gather": {"ms_max_rank": ms[1], "tflops_total": tf(ms[1]),
                                         "gather": "one in-place NCCL all_gather of the rank-major buffer the GEMM wrote into",
                                         "received_bytes_per_rank": recv_bytes, "nvlink_floor_ms": recv_bytes / NVLINK_GBS / 1e6},
            "gemm_fwd": {"ms_max_rank": ms[2], "tflops_total": tf(ms[2])},
            "gemm_wgrad": {"ms_max_rank": ms[3], "tflops_total": tf(ms[3])}}
