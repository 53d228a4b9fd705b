"""token_permute / token_unpermute: MoE token (un)permutation by a routing mask, with autograd.

Operator surface of primus_turbo/pytorch/ops/moe/permutation.py of the reference (token_permute :289-377,
token_unpermute :379-, the fused Functions :26-286).  Only the fused form is provided: it runs on the CUDA kernels of this
package; `fused=False` in the reference is a composition of torch indexing calls, which callers that want it can write
with torch directly.  FP8 payloads (QuantizedTensor inputs) are refused as the reference refuses them
("FP8 is not supported for now").
"""
from typing import Optional, Tuple

import torch

from ...core.quantized_tensor import QuantizedTensor
from ...kernels.moe import permutation_impl as permutation

__all__ = ["token_permute", "token_unpermute"]


class TokenPermuteMaskMap(torch.autograd.Function):
    @staticmethod
    def forward(ctx, inp, routing_map, num_out_tokens, probs, return_tokens_per_expert):
        ctx.inp_shape = inp.shape
        if not inp.numel():
            ctx.probs = probs
            e = lambda: torch.tensor([], device=inp.device)
            return inp, e(), e(), e()
        assert inp.is_cuda and routing_map.is_cuda, "token_permute needs CUDA tensors"
        assert not isinstance(inp, QuantizedTensor), "FP8 is not supported for now."
        assert inp.size(0) == routing_map.size(0), "Permute not possible"
        num_tokens, hidden_size = inp.size()
        num_experts = routing_map.size(1)
        assert num_out_tokens is not None, "num_out_tokens must be provided to the fused permute function."
        row_id_map, tokens_per_experts = permutation.make_row_id_map(routing_map, num_tokens, num_experts,
                                                                     return_tokens_per_expert or num_out_tokens < 0)
        if num_out_tokens < 0:
            num_out_tokens = int(tokens_per_experts.sum().item())
        output, _, permuted_probs = permutation.permute_with_mask_map(inp, row_id_map, probs, None, num_tokens, num_experts,
                                                                      num_out_tokens, hidden_size, None)
        if not output.numel():
            ctx.probs = probs
        ctx.save_for_backward(row_id_map)
        ctx.num_experts, ctx.num_tokens, ctx.hidden_size = num_experts, num_tokens, hidden_size
        return output, row_id_map, permuted_probs, (tokens_per_experts if return_tokens_per_expert else None)

    @staticmethod
    def backward(ctx, permuted_act_grad, _, permuted_probs_grad, __):
        if not permuted_act_grad.numel():
            return (torch.empty(ctx.inp_shape, dtype=permuted_act_grad.dtype, device=permuted_act_grad.device), None, None,
                    ctx.probs, None)
        act_grad = probs_grad = None
        if ctx.needs_input_grad[0]:
            (row_id_map,) = ctx.saved_tensors
            act_grad, probs_grad = permutation.unpermute_with_mask_map(permuted_act_grad, row_id_map, None, permuted_probs_grad,
                                                                       ctx.num_tokens, ctx.num_experts, ctx.hidden_size)
        if not ctx.needs_input_grad[3]:
            probs_grad = None
        return act_grad, None, None, probs_grad, None


class TokenUnpermuteMaskMap(torch.autograd.Function):
    @staticmethod
    def forward(ctx, inp, row_id_map, merging_probs, restore_shape):
        ctx.input_is_empty = inp.numel() == 0
        if ctx.input_is_empty:
            ctx.inp_shape, ctx.merging_probs = inp.shape, merging_probs
            if restore_shape is not None:
                inp = torch.empty(restore_shape, dtype=inp.dtype, device=inp.device)
            return inp
        if restore_shape is None:
            restore_shape = inp.shape
        num_tokens, hidden_size = restore_shape
        num_experts = (row_id_map.size(1) - 1) // 2
        with_probs = merging_probs is not None
        assert inp.is_cuda and row_id_map.is_cuda, "Tensor device needs be CUDA."
        assert not isinstance(inp, QuantizedTensor), "The forward of moe_unpermute does not support FP8."
        out, _ = permutation.unpermute_with_mask_map(inp, row_id_map, merging_probs, None, num_tokens, num_experts, hidden_size)
        if with_probs:
            ctx.save_for_backward(inp, row_id_map, merging_probs)
        else:
            ctx.save_for_backward(row_id_map)
        ctx.num_experts, ctx.num_tokens, ctx.num_permuted_tokens = num_experts, num_tokens, inp.size(0)
        ctx.hidden_size, ctx.with_probs = hidden_size, with_probs
        return out

    @staticmethod
    def backward(ctx, unpermuted_act_grad):
        if ctx.input_is_empty:
            return (torch.empty(ctx.inp_shape, dtype=unpermuted_act_grad.dtype, device=unpermuted_act_grad.device), None,
                    ctx.merging_probs, None)
        act_grad = probs_grad = None
        if ctx.needs_input_grad[0]:
            if ctx.with_probs:
                fwd_input, row_id_map, merging_probs = ctx.saved_tensors
                act_grad, probs_grad = permutation.unpermute_with_mask_map_bwd_with_merging_probs(
                    unpermuted_act_grad, row_id_map, fwd_input, merging_probs, ctx.num_tokens, ctx.num_experts,
                    ctx.num_permuted_tokens, ctx.hidden_size)
            else:
                (row_id_map,) = ctx.saved_tensors
                act_grad, _, _ = permutation.permute_with_mask_map(unpermuted_act_grad, row_id_map, None, None, ctx.num_tokens,
                                                                   ctx.num_experts, ctx.num_permuted_tokens, ctx.hidden_size, None)
        if not ctx.needs_input_grad[2]:
            probs_grad = None
        return act_grad, None, probs_grad, None


def token_permute(inp: torch.Tensor, num_out_tokens: int, probs: Optional[torch.Tensor] = None,
                  routing_map: Optional[torch.Tensor] = None, topk_indices: Optional[torch.Tensor] = None, drop_and_pad: bool = False,
                  fused: bool = True, return_tokens_per_expert: bool = False) -> Tuple[torch.Tensor, Optional[torch.Tensor], torch.Tensor, Optional[torch.Tensor]]:
    """Groups token rows by expert: (permuted [num_out_tokens, H], permuted_probs, row_id_map, tokens_per_expert).

    routing_map [T, E]: non-zero where token t is routed to expert e.  num_out_tokens = -1 counts the routed rows (one host
    read).  Rows of expert 0 come first, tokens keep their order inside an expert."""
    if topk_indices is not None:
        raise NotImplementedError("not support topk_indices")
    if routing_map is None:
        raise ValueError("must be set topk_indices or routing_map")
    if drop_and_pad:
        raise NotImplementedError("drop_and_pad is not provided by the fused permutation")
    output, row_id_map, permuted_probs, tokens_per_experts = TokenPermuteMaskMap.apply(inp, routing_map, num_out_tokens, probs,
                                                                                       return_tokens_per_expert)
    return output, permuted_probs, row_id_map, tokens_per_experts


def token_unpermute(inp: torch.Tensor, sorted_indices: torch.Tensor, merging_probs: Optional[torch.Tensor] = None,
                    restore_shape: Optional[torch.Size] = None, routing_map: Optional[torch.Tensor] = None, fused: bool = True,
                    drop_and_pad: bool = False) -> torch.Tensor:
    """Inverse of token_permute: out[t] = sum over t's experts of (merging_probs[t, e] *) inp[row of (t, e)].
    `sorted_indices` is the row_id_map token_permute returned."""
    if drop_and_pad:
        raise NotImplementedError("drop_and_pad is not provided by the fused permutation")
    return TokenUnpermuteMaskMap.apply(inp, sorted_indices, merging_probs, restore_shape)
