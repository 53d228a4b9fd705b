"""Single-box partitioner for the low-precision GEMM path: one process per GPU (torch.distributed).

The path shards without any exchange inside the compute: a dense GEMM is split along its output columns (each
rank holds the weight rows of its columns, the activation is replicated), a grouped GEMM by expert (each rank
holds its experts' weights and the token rows routed to them).  The only collective is the optional gather of the
outputs over NCCL / NVLink; column-parallel layers followed by a row-parallel one keep the output sharded and skip
it.  The reference has no multi-GPU code on this path; this module is the B200 addition the build targets.

`op` arguments default to the CUDA operators of this package; the tests of the host logic (shard bounds, row
ranges, gather assembly) run the same classes over gloo with a plain matmul passed as `op`.
"""
from typing import Callable, List, Optional, Tuple

import torch
import torch.distributed as dist


def column_shard(n: int, world: int, rank: int, align: int = 128) -> Tuple[int, int]:
    """[lo, hi) of output columns owned by `rank`: contiguous, multiples of `align` (so that 128 x 128 and MX scale
    tiles never straddle a shard), as even as that allows; trailing ranks may own nothing when n is small."""
    blocks = (n + align - 1) // align
    base, extra = divmod(blocks, world)
    lo_b = rank * base + min(rank, extra)
    hi_b = lo_b + base + (1 if rank < extra else 0)
    return min(lo_b * align, n), min(hi_b * align, n)


def expert_shard(num_experts: int, world: int, rank: int) -> Tuple[int, int]:
    """[lo, hi) of experts owned by `rank` (contiguous, as even as possible)."""
    base, extra = divmod(num_experts, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def _world(group) -> Tuple[int, int]:
    if not dist.is_available() or not dist.is_initialized():
        return 1, 0
    return dist.get_world_size(group), dist.get_rank(group)


class ColumnShardedLinear:
    """y = x . W^T with W [N, K] sharded by rows (= output columns) across the ranks of `group`.

    Each rank is built from the full weight (it keeps only its rows) or directly from its shard.  forward() returns
    the local columns [M, hi - lo]; gather() assembles the full [M, N] on every rank (one all_gather).
    """

    def __init__(self, n_total: int, weight_shard: torch.Tensor, group=None, op: Optional[Callable] = None, config=None):
        self.group = group
        self.world, self.rank = _world(group)
        self.n_total = n_total
        self.lo, self.hi = column_shard(n_total, self.world, self.rank)
        assert weight_shard.shape[0] == self.hi - self.lo, "weight shard does not match this rank's column range"
        self.weight = weight_shard
        self.config = config
        self._op = op

    @classmethod
    def from_full_weight(cls, weight: torch.Tensor, group=None, op=None, config=None):
        world, rank = _world(group)
        lo, hi = column_shard(weight.shape[0], world, rank)
        return cls(weight.shape[0], weight[lo:hi].contiguous(), group, op, config)

    def _gemm(self, x):
        if self._op is not None:
            return self._op(x, self.weight)
        from ..ops.gemm_fp8 import gemm_fp8
        return gemm_fp8(x, self.weight, trans_b=True, config=self.config)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if self.hi == self.lo:
            return x.new_zeros((x.shape[0], 0))
        return self._gemm(x)

    def gather(self, y_local: torch.Tensor) -> torch.Tensor:
        """[M, n_local] on every rank -> [M, N] on every rank."""
        if self.world == 1:
            return y_local
        M = y_local.shape[0]
        widths = [column_shard(self.n_total, self.world, r) for r in range(self.world)]
        wmax = max(h - l for l, h in widths)
        # gather transposed so that each rank contributes a contiguous row block of y^T
        send = y_local.new_zeros((wmax, M))
        send[: self.hi - self.lo] = y_local.t()
        recv = y_local.new_empty((self.world * wmax, M))
        dist.all_gather_into_tensor(recv, send, group=self.group)
        parts = [recv[r * wmax: r * wmax + (h - l)] for r, (l, h) in enumerate(widths)]
        return torch.cat(parts, dim=0).t().contiguous()


class ExpertShardedGroupedLinear:
    """Grouped GEMM with the experts sharded across ranks: rank r owns experts [g_lo, g_hi) and, because groups are
    contiguous in the packed token layout, the token rows [offs[g_lo], offs[g_hi]).  Token placement (dispatch) is the
    caller's business; forward() takes this rank's rows only.
    """

    def __init__(self, num_experts: int, weight_shard: torch.Tensor, group=None, op: Optional[Callable] = None, config=None):
        self.group = group
        self.world, self.rank = _world(group)
        self.num_experts = num_experts
        self.g_lo, self.g_hi = expert_shard(num_experts, self.world, self.rank)
        assert weight_shard.shape[0] == self.g_hi - self.g_lo, "weight shard does not match this rank's experts"
        self.weight = weight_shard
        self.config = config
        self._op = op

    @classmethod
    def from_full_weight(cls, weight: torch.Tensor, group=None, op=None, config=None):
        world, rank = _world(group)
        lo, hi = expert_shard(weight.shape[0], world, rank)
        return cls(weight.shape[0], weight[lo:hi].contiguous(), group, op, config)

    def local_rows(self, group_lens_all: List[int]) -> Tuple[int, int]:
        """Row range of the packed token matrix that belongs to this rank's experts."""
        start = sum(group_lens_all[: self.g_lo])
        return start, start + sum(group_lens_all[self.g_lo: self.g_hi])

    def forward(self, x_local: torch.Tensor, group_lens_local: torch.Tensor) -> torch.Tensor:
        if self._op is not None:
            return self._op(x_local, self.weight, group_lens_local)
        from ..ops.grouped_gemm_fp8 import grouped_gemm_fp8
        return grouped_gemm_fp8(x_local, self.weight, group_lens_local, trans_b=True, config=self.config)

    def gather(self, y_local: torch.Tensor, group_lens_all: List[int]) -> torch.Tensor:
        """Concatenates every rank's rows in expert order on every rank (padded all_gather)."""
        if self.world == 1:
            return y_local
        rows = []
        for r in range(self.world):
            lo, hi = expert_shard(self.num_experts, self.world, r)
            rows.append(sum(group_lens_all[lo:hi]))
        rmax = max(max(rows), 1)
        send = y_local.new_zeros((rmax, y_local.shape[1]))
        send[: y_local.shape[0]] = y_local
        recv = y_local.new_empty((self.world * rmax, y_local.shape[1]))
        dist.all_gather_into_tensor(recv, send, group=self.group)
        return torch.cat([recv[r * rmax: r * rmax + n] for r, n in enumerate(rows)], dim=0)
