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


def row_balanced_expert_shard(group_lens: List[int], world: int, rank: int, align: int = 128):
    """Shard of `rank` when the packed token rows, not the experts, are split evenly: the rows [R * rank / world,
    R * (rank + 1) / world) of the expert-major layout (cut points rounded to `align` rows inside an expert).  A popular
    expert then straddles two or more ranks, each of which holds a copy of its weights and a slice of its rows, so one hot
    expert (Zipf routing: a fifth of all rows on one of 256 experts) no longer decides the step time.

    Returns (g_lo, g_hi, local_group_lens): the experts [g_lo, g_hi) this rank touches and how many rows of each."""
    offs = [0]
    for n in group_lens:
        offs.append(offs[-1] + int(n))
    total = offs[-1]

    def cut(r):
        if r <= 0:
            return 0
        if r >= world:
            return total
        c = total * r // world
        g = max(0, min(len(group_lens) - 1, _last_leq(offs, c)))
        inside = c - offs[g]
        return min(offs[g] + (inside + align // 2) // align * align, offs[g + 1])

    lo, hi = cut(rank), cut(rank + 1)
    if hi <= lo:
        return 0, 0, []
    g_lo = _last_leq(offs, lo)
    while g_lo < len(group_lens) and offs[g_lo + 1] <= lo:
        g_lo += 1
    g_hi = g_lo
    lens = []
    while g_hi < len(group_lens) and offs[g_hi] < hi:
        lens.append(min(offs[g_hi + 1], hi) - max(offs[g_hi], lo))
        g_hi += 1
    return g_lo, g_hi, lens


def _last_leq(offs: List[int], v: int) -> int:
    """Largest g with offs[g] <= v (offs ascending, offs[0] = 0)."""
    lo, hi = 0, len(offs) - 2
    while lo < hi:
        mid = (lo + hi + 1) // 2
        if offs[mid] <= v:
            lo = mid
        else:
            hi = mid - 1
    return lo


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
        """[M, n_local] on every rank -> [M, N] on every rank.

        Equal shards (the usual case: N / world a multiple of 128) are gathered as rank-major blocks
        [world, M, n_local] by one all_gather and returned as a permuted VIEW of that buffer ([M, world, n_local]
        flattened to [M, N] is not contiguous; consumers that need contiguity call .contiguous() themselves).
        Ragged shards go through a padded gather of the transposed shard."""
        if self.world == 1:
            return y_local
        M = y_local.shape[0]
        widths = [column_shard(self.n_total, self.world, r) for r in range(self.world)]
        if len({h - l for l, h in widths}) == 1:
            n_local = self.hi - self.lo
            recv = y_local.new_empty((self.world * M, n_local))
            dist.all_gather_into_tensor(recv, y_local.contiguous(), group=self.group)
            return recv.view(self.world, M, n_local).permute(1, 0, 2).reshape(M, self.world * n_local)
        wmax = max(h - l for l, h in widths)
        # gather transposed so that each rank contributes a contiguous row block of y^T
        send = y_local.new_zeros((wmax, M))
        send[: self.hi - self.lo] = y_local.t()
        recv = y_local.new_empty((self.world * wmax, M))
        dist.all_gather_into_tensor(recv, send, group=self.group)
        parts = [recv[r * wmax: r * wmax + (h - l)] for r, (l, h) in enumerate(widths)]
        return torch.cat(parts, dim=0).t().contiguous()

    def gather_buffer(self, M: int, dtype, device) -> torch.Tensor:
        """Rank-major gather buffer [world, M, n_local] for equal shards; forward_into() lets the GEMM write this
        rank's block in place, so the gather needs no send copy."""
        return torch.empty((self.world, M, self.hi - self.lo), dtype=dtype, device=device)

    def forward_into(self, x: torch.Tensor, buf: torch.Tensor) -> torch.Tensor:
        """forward() whose result lands in this rank's block of a gather_buffer().  Without autograd and with the MX
        recipe only the row-wise quantized copies are made (the transposed ones exist for backward) and the GEMM
        writes the block itself; other recipes (and the `op` hook) run forward() and copy."""
        slot = buf[self.rank]
        from ..core.low_precision import ScalingGranularity, ScalingRecipe
        cfg = self.config
        if self._op is None and cfg is not None and cfg.granularity == ScalingGranularity.MX_BLOCKWISE and not torch.is_grad_enabled():
            from ..kernels.gemm.gemm_fp8_impl import gemm_fp8_impl
            from ..kernels.quantization.quantization_impl import quantize_mxfp8_impl
            from ..ops.utils import _get_fp8_dtype
            dt = _get_fp8_dtype(cfg.format, True)
            two_d = ScalingRecipe(use_2d_block=True)
            a_row, a_s = quantize_mxfp8_impl(x, dt, 1, cfg.block_size)
            b_row, b_s = quantize_mxfp8_impl(self.weight, dt, 1, cfg.block_size, scaling_recipe=two_d)
            gemm_fp8_impl(a_row, a_s, False, b_row, b_s, True, slot.dtype, False, cfg.granularity, out=slot)
        else:
            slot.copy_(self.forward(x))
        return slot

    def gather_in_place(self, buf: torch.Tensor) -> torch.Tensor:
        """All-gathers `buf` ([world, M, n_local], this rank's block already written by the caller) in place."""
        if self.world > 1:
            dist.all_gather_into_tensor(buf.view(-1, buf.shape[-1]), buf[self.rank], group=self.group)
        return buf

    # ---- backward, each GEMM sharded along ITS OWN output columns so that no reduction is needed:
    #   wgrad  dW[lo:hi]      = dY[:, lo:hi]^T . X        (the columns of dY this rank produced in forward; stays sharded)
    #   dgrad  dX[:, k0:k1]   = dY . W[:, k0:k1]          (needs the full dY and a K-slice of the full weight)
    def wgrad(self, x: torch.Tensor, dy_local: torch.Tensor, op: Optional[Callable] = None) -> torch.Tensor:
        """[n_local, K] gradient of this rank's weight rows; `op(dy_local, x)` defaults to the FP8 operator's own
        backward (autograd through forward())."""
        if op is not None:
            return op(dy_local, x)
        w = self.weight.detach().requires_grad_(True)
        from ..ops.gemm_fp8 import gemm_fp8
        y = gemm_fp8(x, w, trans_b=True, config=self.config)
        (gw,) = torch.autograd.grad(y, w, dy_local)
        return gw

    @staticmethod
    def dgrad_shard(k_total: int, world: int, rank: int) -> Tuple[int, int]:
        """[k0, k1) of input features whose gradient `rank` computes."""
        return column_shard(k_total, world, rank)

    def dgrad(self, dy_full: torch.Tensor, weight_kslice: torch.Tensor, op: Optional[Callable] = None) -> torch.Tensor:
        """dX[:, k0:k1] = dY [M, N] . W[:, k0:k1] for this rank's K-slice of the FULL weight ([N, k1 - k0])."""
        if op is not None:
            return op(dy_full, weight_kslice)
        from ..ops.gemm_fp8 import gemm_fp8
        return gemm_fp8(dy_full, weight_kslice, trans_b=False, config=self.config)


class ExpertShardedGroupedLinear:
    """Grouped GEMM with the experts sharded across ranks: rank r owns experts [g_lo, g_hi) and, because groups are
    contiguous in the packed token layout, the token rows [offs[g_lo], offs[g_hi]).  Token placement (dispatch) is the
    caller's business; forward() takes this rank's rows only.
    """

    def __init__(self, num_experts: int, weight_shard: torch.Tensor, group=None, op: Optional[Callable] = None, config=None,
                 cache_quantized_weight: bool = False, experts: Optional[Tuple[int, int]] = None):
        """`experts` = (g_lo, g_hi) overrides the even split by expert count, e.g. with the range
        row_balanced_expert_shard() gives (then several ranks may hold the same popular expert and split its rows)."""
        self.group = group
        self.world, self.rank = _world(group)
        self.num_experts = num_experts
        self.g_lo, self.g_hi = expert_shard(num_experts, self.world, self.rank) if experts is None else experts
        assert weight_shard.shape[0] == self.g_hi - self.g_lo, "weight shard does not match this rank's experts"
        self.weight = weight_shard
        self.config = config
        self._op = op
        self._qcache = None
        if cache_quantized_weight:
            from ..modules._weight_cache import QuantizedWeightCache
            self._qcache = QuantizedWeightCache()

    @classmethod
    def from_full_weight(cls, weight: torch.Tensor, group=None, op=None, config=None, cache_quantized_weight=False):
        world, rank = _world(group)
        lo, hi = expert_shard(weight.shape[0], world, rank)
        return cls(weight.shape[0], weight[lo:hi].contiguous(), group, op, config, cache_quantized_weight)

    def local_rows(self, group_lens_all: List[int]) -> Tuple[int, int]:
        """Row range of the packed token matrix that belongs to this rank's experts."""
        start = sum(group_lens_all[: self.g_lo])
        return start, start + sum(group_lens_all[self.g_lo: self.g_hi])

    def forward(self, x_local: torch.Tensor, group_lens_local: torch.Tensor) -> torch.Tensor:
        if self._op is not None:
            return self._op(x_local, self.weight, group_lens_local)
        from ..ops.grouped_gemm_fp8 import grouped_gemm_fp8
        w = self.weight
        if self._qcache is not None:   # the experts' quantized copies are reused until the weight changes
            from ..ops.utils import _get_fp8_dtype
            w = self._qcache.get(self.weight, _get_fp8_dtype(self.config.format, True), self.config,
                                 need_transpose=False)
        return grouped_gemm_fp8(x_local, w, group_lens_local, trans_b=True, config=self.config)

    def gather_rows(self, y_local: torch.Tensor, rows: List[int]) -> torch.Tensor:
        """Concatenates every rank's rows in rank order on every rank; rows[r] = row count of rank r (padded all_gather)."""
        if self.world == 1:
            return y_local
        rmax = max(max(rows), 1)
        send = y_local.new_zeros((rmax, y_local.shape[1]))
        send[: y_local.shape[0]] = y_local
        recv = y_local.new_empty((self.world * rmax, y_local.shape[1]))
        dist.all_gather_into_tensor(recv, send, group=self.group)
        return torch.cat([recv[r * rmax: r * rmax + n] for r, n in enumerate(rows)], dim=0)

    def gather(self, y_local: torch.Tensor, group_lens_all: List[int]) -> torch.Tensor:
        """Concatenates every rank's rows in expert order on every rank (padded all_gather); for the even split by
        expert count."""
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
