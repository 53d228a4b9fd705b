"""The partitioner with the real CUDA operators on 2 GPUs (NCCL): column-sharded MX GEMM and expert-sharded
blockwise grouped GEMM reproduce the single-GPU results.  Skipped when fewer than 2 GPUs are visible."""
import os
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu


def _worker(rank, world, port, root):
    import torch.distributed as dist
    sys.path.insert(0, root)
    sys.path.insert(0, os.path.join(root, "primus-turbo_b200"))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        import primus_turbo.pytorch as turbo
        from primus_turbo.pytorch.core.low_precision import Float8QuantConfig, Format, ScaleDtype, ScalingGranularity
        from primus_turbo.pytorch.dist import ColumnShardedLinear, ExpertShardedGroupedLinear
        g = torch.Generator().manual_seed(0)
        x = torch.randn(512, 1024, generator=g).to(torch.bfloat16).cuda()
        w = (0.02 * torch.randn(1536, 1024, generator=g)).to(torch.bfloat16).cuda()
        cfg = Float8QuantConfig(format=Format.E4M3, granularity=ScalingGranularity.MX_BLOCKWISE, scale_dtype=ScaleDtype.E8M0,
                                block_size=32)
        with torch.no_grad():
            lin = ColumnShardedLinear.from_full_weight(w, config=cfg)
            y = lin.gather(lin.forward(x))
            full = turbo.ops.gemm_fp8(x, w, trans_b=True, config=cfg)
        assert torch.equal(y, full), "column-sharded MX GEMM differs from the unsharded one"
        lens = [100, 0, 300, 29, 64, 7, 128, 256]
        we = (0.02 * torch.randn(8, 384, 512, generator=g)).to(torch.bfloat16).cuda()
        xe = torch.randn(sum(lens), 512, generator=g).to(torch.bfloat16).cuda()
        bcfg = Float8QuantConfig(format=Format.E4M3, granularity=ScalingGranularity.BLOCKWISE, block_size=128)
        with torch.no_grad():
            ex = ExpertShardedGroupedLinear.from_full_weight(we, config=bcfg)
            r0, r1 = ex.local_rows(lens)
            y_loc = ex.forward(xe[r0:r1].contiguous(), torch.tensor(lens[ex.g_lo:ex.g_hi], dtype=torch.int64, device="cuda"))
            y_all = ex.gather(y_loc, lens)
            full = turbo.ops.grouped_gemm_fp8(xe, we, torch.tensor(lens, dtype=torch.int64, device="cuda"), trans_b=True, config=bcfg)
        assert torch.equal(y_all, full), "expert-sharded grouped GEMM differs from the unsharded one"
        # FP8 all-to-all: unequal splits, forward + backward; the wire format costs at most the e4m3 / e5m2 rounding
        from primus_turbo.pytorch.dist import FP8AllToAll
        tcfg = Float8QuantConfig(format=Format.HYBRID, granularity=ScalingGranularity.TENSORWISE)
        in_splits = [3, 5] if rank == 0 else [4, 2]
        out_splits = [3, 4] if rank == 0 else [5, 2]
        gen = torch.Generator().manual_seed(10 + rank)
        t = torch.randn(sum(in_splits), 256, generator=gen).to(torch.bfloat16).cuda().requires_grad_()
        got = FP8AllToAll.apply(dist.group.WORLD, t, out_splits, in_splits, True, True, tcfg)
        want = torch.empty((sum(out_splits), 256), dtype=torch.bfloat16, device="cuda")
        dist.all_to_all_single(want, t.detach(), output_split_sizes=out_splits, input_split_sizes=in_splits)
        assert got.shape == want.shape
        assert float((got.float() - want.float()).norm() / want.float().norm()) < 0.05
        got.backward(torch.ones_like(got))
        assert t.grad.shape == t.shape and torch.allclose(t.grad.float(), torch.ones_like(t.grad).float(), atol=0.07)
        plain = FP8AllToAll.apply(dist.group.WORLD, t.detach(), out_splits, in_splits, False, False, tcfg)
        assert torch.equal(plain, want)
        torch.cuda.synchronize()
        dist.barrier()
    finally:
        dist.destroy_process_group()


def test_partitioner_two_gpus():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    import torch.multiprocessing as mp
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    mp.spawn(_worker, args=(2, 29731, root), nprocs=2, join=True)
