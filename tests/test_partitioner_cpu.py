"""Host logic of the single-box partitioner on CPU ranks (gloo, world_size 2 and 3): shard bounds, row ranges and
the gather assembly, with a plain matmul standing in for the CUDA operators (the `op` hook exists for this)."""
import os

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from primus_turbo.pytorch.dist.partitioner import (ColumnShardedLinear, ExpertShardedGroupedLinear, column_shard,
                                                    expert_shard, row_balanced_expert_shard)


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


def test_row_balanced_expert_shard_covers_every_row_once():
    import numpy as np
    rng = np.random.default_rng(0)
    for lens in ([27140, 0, 3, 500, 128, 0, 9000, 1], [5] * 7, [0, 0, 4096], list(rng.integers(0, 3000, size=64))):
        lens = [int(v) for v in lens]
        for world in (1, 2, 3, 4, 8):
            cover = [0] * len(lens)
            rows = []
            prev_hi = 0
            for r in range(world):
                g_lo, g_hi, local = row_balanced_expert_shard(lens, world, r)
                assert len(local) == g_hi - g_lo and all(n >= 0 for n in local)
                if local:
                    assert g_lo >= max(prev_hi - 1, 0)      # ranks walk the experts in order; neighbours may share one
                    prev_hi = g_hi
                for i, n in enumerate(local):
                    cover[g_lo + i] += n
                rows.append(sum(local))
            assert cover == lens
            if sum(lens) >= 128 * world * 8:
                assert max(rows) <= sum(lens) / world + 128  # balanced to within one alignment unit


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
        # equal shards: the rank-major buffer is gathered in place and viewed as [M, N]
        w2 = torch.randn(128 * world * 2, 64, generator=g)
        lin2 = ColumnShardedLinear.from_full_weight(w2, op=lambda a, b: a @ b.t())
        buf = lin2.gather_buffer(x.shape[0], x.dtype, x.device)
        lin2.forward_into(x, buf)
        full = lin2.gather_in_place(buf).permute(1, 0, 2).reshape(x.shape[0], -1)
        assert torch.allclose(full, x @ w2.t(), atol=1e-5), "in-place gather differs"
        assert torch.allclose(lin2.gather(lin2.forward(x)), x @ w2.t(), atol=1e-5), "equal-shard gather differs"
        # backward shards: each GEMM is split along its own output columns, so no rank needs a reduction
        dy = torch.randn(37, w2.shape[0], generator=g)
        gw = lin2.wgrad(x, dy[:, lin2.lo:lin2.hi], op=lambda d, a: d.t() @ a)
        assert torch.allclose(gw, (dy.t() @ x)[lin2.lo:lin2.hi], atol=1e-4), "sharded wgrad differs"
        k0, k1 = lin2.dgrad_shard(64, world, dist.get_rank())
        gx = lin2.dgrad(dy, w2[:, k0:k1], op=lambda d, ws: d @ ws)
        assert torch.allclose(gx, (dy @ w2)[:, k0:k1], atol=1e-4), "sharded dgrad differs"
        dist.barrier()
    finally:
        dist.destroy_process_group()


def _failing_worker(rank, world, port, out_dir):
    """Rank 1 raises before the collective; rank 0 must get an error from its all_gather (not hang) and say so."""
    import datetime
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=10))
    w = torch.randn(256, 16)
    lin = ColumnShardedLinear.from_full_weight(w, op=lambda a, b: a @ b.t())
    y = lin.forward(torch.randn(4, 16))
    dist.barrier()
    if rank == 1:
        raise RuntimeError("injected failure before the gather")
    try:
        lin.gather(y)
        outcome = "gather returned"
    except Exception as exc:  # noqa: BLE001
        outcome = "gather failed: " + type(exc).__name__
    with open(os.path.join(out_dir, "rank0.txt"), "w") as f:
        f.write(outcome)


def test_rank_that_raises_before_the_collective(tmp_path):
    """Host-side failure detection: the surviving rank's collective ends with an error within the group's timeout."""
    ctx = mp.get_context("spawn")
    port = 29900 + (os.getpid() % 90)
    procs = [ctx.Process(target=_failing_worker, args=(r, 2, port, str(tmp_path))) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=90)
    assert all(not p.is_alive() for p in procs), "a rank hung after its peer failed"
    assert procs[1].exitcode != 0
    assert (tmp_path / "rank0.txt").read_text().startswith("gather failed"), (tmp_path / "rank0.txt").read_text()


@pytest.mark.parametrize("world", [2, 3])
def test_partitioner_over_gloo(world):
    port = 29600 + world + (os.getpid() % 200)
    mp.spawn(_worker, args=(world, port), nprocs=world, join=True)
