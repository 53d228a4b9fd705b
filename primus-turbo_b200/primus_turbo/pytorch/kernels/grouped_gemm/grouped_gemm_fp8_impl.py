"""Grouped FP8 / MXFP8 GEMMs over the C ABI.

Call shapes follow primus_turbo::grouped_gemm_fp8_impl, grouped_gemm_fp8_variable_k_impl and
grouped_gemm_fp8_variable_k_accum_impl of the reference
(primus_turbo/pytorch/kernels/grouped_gemm/grouped_gemm_fp8_impl.py:888-1030).  No call synchronises with the host:
group offsets stay on the device.
"""
from typing import Optional

import torch

from ...core.low_precision import ScalingGranularity
from .. import _native as nv
from ..gemm.gemm_fp8_impl import _GRAN, _as_gran


def _ws(gran, rows, N, K, G, mode, device):
    n = nv.lib().pt_gemm_fp8_workspace_bytes(_GRAN[gran], rows, N, K, G, mode, 0)
    return (torch.empty(n, dtype=torch.uint8, device=device) if n else None), n


def grouped_gemm_fp8_impl(a: torch.Tensor, b: torch.Tensor, a_scales: torch.Tensor, b_scales: torch.Tensor,
                          group_lens: torch.Tensor, group_offs: torch.Tensor, trans_a: bool, trans_b: bool,
                          out_dtype: torch.dtype, granularity, num_cu: Optional[int] = None, default_backend: int = 0,
                          maybe_pre_sync: bool = False, group_offs_out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[offs_out[g] : offs_out[g] + len_g] = a[offs[g] : offs[g] + len_g] . op(b[g]).

    a [rows, K] (read at `group_offs`), b [G, N, K] (trans_b) or [G, K, N]; `group_offs_out` (default: group_offs)
    is where each group's rows are written.  The output has a's row count; rows past the last group are zero.
    """
    nv.require_cuda(a, b, a_scales, b_scales, group_lens, group_offs)
    assert not trans_a, "grouped GEMM takes a row-major activation (trans_a=False)"
    assert a.dim() == 2 and b.dim() == 3
    gran = _as_gran(granularity)
    G = b.shape[0]
    a = a.contiguous()
    b = b.contiguous()
    rows, K = a.shape
    N = b.shape[1] if trans_b else b.shape[2]
    offs_read = group_offs.to(torch.int64).contiguous()
    offs_write = offs_read if group_offs_out is None else group_offs_out.to(torch.int64).contiguous()
    # rows past the last group stay zero: only that tail is cleared (its first row is read on the device)
    out = torch.empty((rows, N), dtype=out_dtype, device=a.device)
    with nv.on_device(a.device):
        nv.check(nv.lib().pt_zero_rows_from(nv.ptr(out), rows, N * out.element_size(), nv.ptr(offs_write[G:]), nv.stream(a.device)),
                 "zero_rows_from")
    st = nv.status_word(a.device)
    max_ctas = int(num_cu) if num_cu else 0
    lib = nv.lib()
    with nv.on_device(a.device):
        if gran == ScalingGranularity.BLOCKWISE:
            a_s = a_scales.to(torch.float32).contiguous()
            b_s = b_scales.to(torch.float32).contiguous()
            kb = (K + 127) // 128
            # activation scales: transposed [K/128, rows] (fused grouped quantizer) or row-major [rows, K/128]
            if a_s.shape[0] == kb and a_s.shape[1] == rows:
                a_desc = (0, 1, rows)
            else:
                assert tuple(a_s.shape) == (rows, kb), f"unexpected activation scale shape {tuple(a_s.shape)}"
                a_desc = (0, kb, 1)
            if trans_b:   # b [G, N, K], tiles [G, N/128, K/128]
                b_desc = (7, b_s.shape[2], 1, b_s.shape[1] * b_s.shape[2])
                b_mn, b_rows, b_cols = 0, G * N, K
            else:         # b [G, K, N] read in place as an MN-major operand, tiles [G, K/128, N/128]
                b_desc = (7, 1, b_s.shape[2], b_s.shape[1] * b_s.shape[2])
                b_mn, b_rows, b_cols = 1, G * K, N
                assert K % 128 == 0 or G == 1, "a [G, K, N] weight needs K % 128 == 0"
            nv.check(lib.pt_grouped_gemm_fp8_blockwise(
                nv.ptr(a), nv.fmt_code(a.dtype), 0, rows, K, nv.ptr(a_s), *a_desc,
                nv.ptr(b), nv.fmt_code(b.dtype), b_mn, b_rows, b_cols, nv.ptr(b_s), *b_desc,
                nv.ptr(out), nv.src_code(out_dtype), rows, N, K, nv.ptr(offs_read), nv.ptr(offs_write), None, G, 0.0,
                max_ctas, nv.ptr(st), nv.stream(a.device)), "grouped_gemm_fp8_blockwise")
            nv.poll_status(out.device)
            return out
        assert trans_b, "this granularity takes b as [G, N, K] (trans_b=True)"
        if gran in (ScalingGranularity.TENSORWISE, ScalingGranularity.ROWWISE):
            a_s = a_scales.to(torch.float32).reshape(-1).contiguous()
            b_s = b_scales.to(torch.float32).reshape(-1).contiguous()
        else:
            a_s, b_s = a_scales.contiguous(), b_scales.contiguous()
        ws, ws_bytes = _ws(gran, rows, N, K, G, 1, a.device)
        nv.check(lib.pt_grouped_gemm_fp8(nv.ptr(a), nv.ptr(a_s), nv.fmt_code(a.dtype), nv.ptr(b), nv.ptr(b_s),
                                         nv.fmt_code(b.dtype), nv.ptr(out), nv.src_code(out_dtype), _GRAN[gran], rows, rows, N, K,
                                         nv.ptr(offs_read), nv.ptr(offs_write), G, 0.0, 0, max_ctas, nv.ptr(ws), ws_bytes,
                                         nv.ptr(st), nv.stream(a.device)), "grouped_gemm_fp8")
    nv.poll_status(out.device)
    return out


def _variable_k(a, b, a_scales, b_scales, group_lens, group_offs, trans_a, trans_b, trans_c, out_dtype, granularity, num_cu,
                out=None):
    nv.require_cuda(a, b, a_scales, b_scales, group_lens, group_offs)
    gran = _as_gran(granularity)
    G = group_lens.numel()
    k_offs = group_offs.to(torch.int64).contiguous()
    a, b = a.contiguous(), b.contiguous()
    st = nv.status_word(a.device)
    max_ctas = int(num_cu) if num_cu else 0
    beta = 0.0 if out is None else 1.0
    lib = nv.lib()
    with nv.on_device(a.device):
        if gran == ScalingGranularity.BLOCKWISE:
            # a [T, Ka], b [T, Nb] token-major (T = padded tokens); C[g] = a[seg]^T . b[seg] -> [Ka, Nb] (or transposed)
            assert trans_a and not trans_b, "blockwise variable-K takes token-major operands (trans_a=True, trans_b=False)"
            lhs, lhs_s, rhs, rhs_s = (b, b_scales, a, a_scales) if trans_c else (a, a_scales, b, b_scales)
            T, R = lhs.shape
            Nn = rhs.shape[1]
            lhs_s = lhs_s.to(torch.float32).contiguous()
            rhs_s = rhs_s.to(torch.float32).contiguous()
            if out is None:
                out = torch.empty((G, R, Nn), dtype=out_dtype, device=a.device)
            nv.check(lib.pt_grouped_gemm_fp8_blockwise(
                nv.ptr(lhs), nv.fmt_code(lhs.dtype), 1, T, R, nv.ptr(lhs_s), 0, 1, R,
                nv.ptr(rhs), nv.fmt_code(rhs.dtype), 1, T, Nn, nv.ptr(rhs_s), 0, 1, Nn, 0,
                nv.ptr(out), nv.src_code(out.dtype), R, Nn, T, None, None, nv.ptr(k_offs), G, beta, max_ctas, nv.ptr(st),
                nv.stream(a.device)), "grouped_gemm_fp8_blockwise_variable_k")
            nv.poll_status(out.device)
            return out
        # K-major operands sharing the padded token axis as contraction: a [Ra, T], b [Rb, T]; C[g] = a[:, seg] . b[:, seg]^T
        assert not trans_a and not trans_b, "variable-K takes [rows, tokens] operands (trans_a=False, trans_b=False)"
        lhs, lhs_s, rhs, rhs_s = (b, b_scales, a, a_scales) if trans_c else (a, a_scales, b, b_scales)
        R, T = lhs.shape
        Nn = rhs.shape[0]
        if gran in (ScalingGranularity.TENSORWISE, ScalingGranularity.ROWWISE):
            lhs_s = lhs_s.to(torch.float32).reshape(-1).contiguous()
            rhs_s = rhs_s.to(torch.float32).reshape(-1).contiguous()
        else:
            lhs_s, rhs_s = lhs_s.contiguous(), rhs_s.contiguous()
        if out is None:
            out = torch.empty((G, R, Nn), dtype=out_dtype, device=a.device)
        ws, ws_bytes = _ws(gran, R, Nn, T, G, 2, a.device)
        nv.check(lib.pt_grouped_gemm_fp8_variable_k(nv.ptr(lhs), nv.ptr(lhs_s), nv.fmt_code(lhs.dtype), nv.ptr(rhs), nv.ptr(rhs_s),
                                                    nv.fmt_code(rhs.dtype), nv.ptr(out), nv.src_code(out.dtype), _GRAN[gran], R, Nn, T,
                                                    nv.ptr(k_offs), G, beta, 0, max_ctas, nv.ptr(ws), ws_bytes, nv.ptr(st),
                                                    nv.stream(a.device)), "grouped_gemm_fp8_variable_k")
    nv.poll_status(out.device)
    return out


def grouped_gemm_fp8_variable_k_impl(a, b, a_scales, b_scales, group_lens, group_offs, trans_a, trans_b, trans_c, out_dtype,
                                     granularity, num_cu=None, default_backend: int = 0):
    """Per group g: C[g] = a[segment g]^T . b[segment g] over the group's (128-padded) token segment -> [G, ., .]."""
    return _variable_k(a, b, a_scales, b_scales, group_lens, group_offs, trans_a, trans_b, trans_c, out_dtype, granularity, num_cu)


def grouped_gemm_fp8_variable_k_accum_impl(a, b, a_scales, b_scales, group_lens, group_offs, trans_a, trans_b, trans_c, out,
                                           granularity, num_cu=None, default_backend: int = 0):
    """out[g] += ... (beta = 1); `out` is modified in place and returned."""
    return _variable_k(a, b, a_scales, b_scales, group_lens, group_offs, trans_a, trans_b, trans_c, out.dtype, granularity,
                       num_cu, out=out)
