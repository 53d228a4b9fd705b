"""Host logic of the single-box partitioner on CPU ranks (gloo, world_size 2 and 3): shard bounds, row ranges and
the gather assembly, with a plain matmul standing in for the CUDA operators (the `op` hook exists for this)."""
import os

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from primus_turbo.pytorch.dist.partitioner import (ColumnShardedLinear, ExpertShardedGroupedLinear, column_shard,
                                                    expert_shard)


def test_column_shard_bounds():
    for n in (14336, 4096, 100, 128, 129, 28672):
        for world in (1, 2, 3, 4, 8):
            spans = [column_shard(n, world, r) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == n
            for (l0, h0), (l1, h1) in zip(spans, spans[1:]):
                assert h0 == l1 and l0 <= h0
            assert all(l % 128 == 0 for l, h in spans if h > l)
    assert column_shard(14336, 8, 3) == (3 * 1792, 4 * 1792)


def test_expert_shard_bounds():
    assert [expert_shard(256, 8, r) for r in range(8)] == [(32 * r, 32 * r + 32) for r in range(8)]
    spans = [expert_shard(10, 4, r) for r in range(4)]
    assert spans == [(0, 3), (3, 6), (6, 8), (8, 10)]


def _grouped_ref(x, w, lens):
    outs, s = [], 0
    for g, n in enumerate(lens.tolist()):
        outs.append(x[s:s + n] @ w[g].t())
        s += n
    return torch.cat(outs) if outs else x.new_zeros((0, w.shape[1]))


def _worker(rank, world, port):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        g = torch.Generator().manual_seed(0)
        x = torch.randn(37, 64, generator=g)
        w = torch.randn(300, 64, generator=g)
        lin = ColumnShardedLinear.from_full_weight(w, op=lambda a, b: a @ b.t())
        y = lin.gather(lin.forward(x))
        assert torch.allclose(y, x @ w.t(), atol=1e-5), "column-sharded gather does not reproduce the full product"
        # experts: 5 experts over `world` ranks, ragged and empty groups
        lens = [7, 0, 12, 3, 9]
        we = torch.randn(5, 48, 64, generator=g)
        xe = torch.randn(sum(lens), 64, generator=g)
        ex = ExpertShardedGroupedLinear.from_full_weight(we, op=_grouped_ref)
        r0, r1 = ex.local_rows(lens)
        y_loc = ex.forward(xe[r0:r1], torch.tensor(lens[ex.g_lo:ex.g_hi]))
        y_all = ex.gather(y_loc, lens)
        assert torch.allclose(y_all, _grouped_ref(xe, we, torch.tensor(lens)), atol=1e-5), "expert gather differs"
        # a rank that raises before the collective must not hang the others: checked on the host with a barrier timeout
        dist.barrier()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_partitioner_over_gloo(world):
    port = 29600 + world + (os.getpid() % 200)
    mp.spawn(_worker, args=(world, port), nprocs=world, join=True)
