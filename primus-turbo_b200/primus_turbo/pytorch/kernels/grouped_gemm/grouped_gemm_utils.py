"""Group offset helpers (primus_turbo/pytorch/kernels/grouped_gemm/grouped_gemm_utils.py:28-34 of the reference)."""
import torch

from .. import _native as nv


def group_offs_from_lens(group_lens: torch.Tensor) -> torch.Tensor:
    """offs[0] = 0, offs[i+1] = sum(lens[:i+1]); int64, computed on the device without a host sync."""
    nv.require_cuda(group_lens)
    lens = group_lens.to(torch.int64).contiguous()
    G = lens.numel()
    offs = torch.empty(G + 1, dtype=torch.int64, device=lens.device)
    with nv.on_device(lens.device):
        nv.check(nv.lib().pt_compute_group_offs(nv.ptr(lens), G, nv.ptr(offs), nv.stream(lens.device)), "compute_group_offs")
    return offs
