"""MoE token permutation over the C ABI: row_id_map construction, permute, unpermute and the backward of the weighted
unpermute.  Same function names and argument order as primus_turbo/triton/moe/permutation.py of the reference."""
from typing import Optional, Tuple

import torch

from .. import _native as nv


def make_row_id_map(routing_map: torch.Tensor, num_tokens: int, num_experts: int, return_tokens_per_expert: bool = True):
    """routing_map [T, E] (bool / int32 / int64) -> (row_id_map int32 [T, 2E + 1], tokens_per_expert int64 [E] or None)."""
    nv.require_cuda(routing_map)
    assert routing_map.dim() == 2 and tuple(routing_map.shape) == (num_tokens, num_experts)
    rm = routing_map.contiguous()
    if rm.dtype not in (torch.bool, torch.int32, torch.int64):
        rm = rm.to(torch.int32)
    row_id_map = torch.empty((num_tokens, 2 * num_experts + 1), dtype=torch.int32, device=rm.device)
    tpe = torch.empty((num_experts,), dtype=torch.int64, device=rm.device)
    lib = nv.lib()
    ws_bytes = lib.pt_moe_row_id_map_workspace_bytes(num_tokens, num_experts)
    ws = torch.empty(max(ws_bytes, 4), dtype=torch.uint8, device=rm.device)
    with nv.on_device(rm.device):
        nv.check(lib.pt_moe_make_row_id_map(nv.ptr(rm), rm.element_size(), num_tokens, num_experts, nv.ptr(row_id_map), nv.ptr(tpe),
                                            nv.ptr(ws), ws_bytes, nv.stream(rm.device)), "moe_make_row_id_map")
    return row_id_map, (tpe if return_tokens_per_expert else None)


def permute_with_mask_map(inp: torch.Tensor, row_id_map: torch.Tensor, probs: Optional[torch.Tensor], scale: Optional[torch.Tensor],
                          num_tokens: int, num_experts: int, num_out_tokens: int, hidden_size: int,
                          scale_hidden_dim: Optional[int] = None) -> Tuple[torch.Tensor, Optional[torch.Tensor], Optional[torch.Tensor]]:
    """(permuted [num_out_tokens, H], permuted_scale or None, permuted_probs [num_out_tokens] or None)."""
    nv.require_cuda(inp, row_id_map, probs, scale)
    inp = inp.contiguous()
    out = torch.empty((num_out_tokens, hidden_size), dtype=inp.dtype, device=inp.device)
    out_probs = None
    if probs is not None:
        probs = probs.contiguous()
        assert tuple(probs.shape) == (num_tokens, num_experts)
        out_probs = torch.empty((num_out_tokens,), dtype=probs.dtype, device=inp.device)
    lib = nv.lib()
    with nv.on_device(inp.device):
        nv.check(lib.pt_moe_permute(nv.ptr(inp.view(torch.uint8)), num_tokens, hidden_size * inp.element_size(), num_experts,
                                    nv.ptr(row_id_map), nv.ptr(probs), 0 if probs is None else probs.element_size(), num_out_tokens,
                                    nv.ptr(out.view(torch.uint8)), nv.ptr(out_probs), nv.stream(inp.device)), "moe_permute")
        out_scale = None
        if scale is not None:   # per-token scale rows of an FP8 payload travel the same way
            scale = scale.contiguous()
            out_scale = torch.empty((num_out_tokens, scale.shape[1]), dtype=scale.dtype, device=inp.device)
            rb = scale.shape[1] * scale.element_size()
            assert rb % 16 == 0, "scale rows must be a multiple of 16 bytes"
            nv.check(lib.pt_moe_permute(nv.ptr(scale.view(torch.uint8)), num_tokens, rb, num_experts, nv.ptr(row_id_map), None, 0,
                                        num_out_tokens, nv.ptr(out_scale.view(torch.uint8)), None, nv.stream(inp.device)), "moe_permute")
    return out, out_scale, out_probs


def unpermute_with_mask_map(inp: torch.Tensor, row_id_map: torch.Tensor, merging_probs: Optional[torch.Tensor],
                            permuted_probs: Optional[torch.Tensor], num_tokens: int, num_experts: int,
                            hidden_size: int) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
    """(unpermuted [T, H], unpermuted_probs [T, E] or None)."""
    nv.require_cuda(inp, row_id_map, merging_probs, permuted_probs)
    inp = inp.contiguous()
    out = torch.empty((num_tokens, hidden_size), dtype=inp.dtype, device=inp.device)
    pd = merging_probs if merging_probs is not None else permuted_probs
    probs_dtype = pd.dtype if pd is not None else torch.float32
    if merging_probs is not None:
        merging_probs = merging_probs.contiguous()
    unp = None
    if permuted_probs is not None:
        permuted_probs = permuted_probs.contiguous().to(probs_dtype)
        unp = torch.empty((num_tokens, num_experts), dtype=probs_dtype, device=inp.device)
    with nv.on_device(inp.device):
        nv.check(nv.lib().pt_moe_unpermute(nv.ptr(inp), nv.src_code(inp.dtype), num_tokens, hidden_size, num_experts, nv.ptr(row_id_map),
                                           nv.ptr(merging_probs), nv.ptr(permuted_probs), nv.src_code(probs_dtype), nv.ptr(out), nv.ptr(unp),
                                           nv.stream(inp.device)), "moe_unpermute")
    return out, unp


def unpermute_with_mask_map_bwd_with_merging_probs(fwd_output_grad: torch.Tensor, row_id_map: torch.Tensor, fwd_input: torch.Tensor,
                                                   merging_probs: torch.Tensor, num_tokens: int, num_experts: int, num_out_tokens: int,
                                                   hidden_size: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """(act_grad [num_out_tokens, H], merging_probs_grad [T, E])."""
    nv.require_cuda(fwd_output_grad, row_id_map, fwd_input, merging_probs)
    g, x, p = fwd_output_grad.contiguous(), fwd_input.contiguous(), merging_probs.contiguous()
    act_grad = torch.zeros((num_out_tokens, hidden_size), dtype=g.dtype, device=g.device)
    probs_grad = torch.empty((num_tokens, num_experts), dtype=p.dtype, device=g.device)
    with nv.on_device(g.device):
        nv.check(nv.lib().pt_moe_unpermute_bwd_with_probs(nv.ptr(g), nv.ptr(x), nv.src_code(g.dtype), num_tokens, hidden_size, num_experts,
                                                          nv.ptr(row_id_map), nv.ptr(p), nv.src_code(p.dtype), nv.ptr(act_grad),
                                                          nv.ptr(probs_grad), nv.stream(g.device)), "moe_unpermute_bwd_with_probs")
    return act_grad, probs_grad
