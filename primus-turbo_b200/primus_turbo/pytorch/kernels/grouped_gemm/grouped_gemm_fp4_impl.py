"""Grouped MXFP4 GEMMs over the C ABI (primus_turbo::grouped_gemm_fp4_impl, _variable_k_impl, _variable_k_accum_impl of the
reference, primus_turbo/pytorch/kernels/grouped_gemm/grouped_gemm_fp4_impl.py:430-)."""
from typing import Optional

import torch

from .. import _native as nv


def grouped_gemm_fp4_impl(a, b, a_scales, b_scales, group_lens, group_offs, trans_a=False, trans_b=True, out_dtype=torch.bfloat16,
                          granularity=None, num_cu: Optional[int] = None, default_backend: int = 0,
                          group_offs_out: Optional[torch.Tensor] = None):
    """a [rows, K/2] packed e2m1 read at `group_offs`, b [G, N, K/2]; output rows written at `group_offs_out`."""
    nv.require_cuda(a, b, a_scales, b_scales, group_lens, group_offs)
    assert not trans_a and trans_b, "MXFP4 grouped GEMM only supports the NT layout"
    a, b = a.contiguous(), b.contiguous()
    G, N = b.shape[0], b.shape[1]
    rows = a.shape[0]
    K = a.view(torch.uint8).shape[1] * 2
    offs_read = group_offs.to(torch.int64).contiguous()
    offs_write = offs_read if group_offs_out is None else group_offs_out.to(torch.int64).contiguous()
    # rows past the last group stay zero: only that tail is cleared (its first row is read on the device)
    out = torch.empty((rows, N), dtype=out_dtype, device=a.device)
    with nv.on_device(a.device):
        nv.check(nv.lib().pt_zero_rows_from(nv.ptr(out), rows, N * out.element_size(), nv.ptr(offs_write[G:]), nv.stream(a.device)),
                 "zero_rows_from")
    lib = nv.lib()
    ws_bytes = lib.pt_gemm_fp4_workspace_bytes(rows, N, K, G, 1, 0)
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device=a.device)
    st = nv.status_word(a.device)
    with nv.on_device(a.device):
        nv.check(lib.pt_grouped_gemm_fp4(nv.ptr(a), nv.ptr(a_scales.contiguous()), nv.ptr(b), nv.ptr(b_scales.contiguous()), nv.ptr(out),
                                         nv.src_code(out_dtype), rows, rows, N, K, nv.ptr(offs_read), nv.ptr(offs_write), G, 0.0, 0,
                                         int(num_cu) if num_cu else 0, nv.ptr(ws), ws_bytes, nv.ptr(st), nv.stream(a.device)),
                 "grouped_gemm_fp4")
    nv.poll_status(out.device)
    return out


def _variable_k(a, b, a_scales, b_scales, group_lens, group_offs, out_dtype, num_cu, out=None):
    nv.require_cuda(a, b, a_scales, b_scales, group_lens, group_offs)
    a, b = a.contiguous(), b.contiguous()
    G = group_lens.numel()
    M, N = a.shape[0], b.shape[0]
    T = a.view(torch.uint8).shape[1] * 2
    k_offs = group_offs.to(torch.int64).contiguous()
    beta = 0.0
    if out is None:
        out = torch.empty((G, M, N), dtype=out_dtype, device=a.device)
    else:
        beta = 1.0
    lib = nv.lib()
    ws_bytes = lib.pt_gemm_fp4_workspace_bytes(M, N, T, G, 2, 0)
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device=a.device)
    st = nv.status_word(a.device)
    with nv.on_device(a.device):
        nv.check(lib.pt_grouped_gemm_fp4_variable_k(nv.ptr(a), nv.ptr(a_scales.contiguous()), nv.ptr(b), nv.ptr(b_scales.contiguous()),
                                                    nv.ptr(out), nv.src_code(out.dtype), M, N, T, nv.ptr(k_offs), G, beta, 0,
                                                    int(num_cu) if num_cu else 0, nv.ptr(ws), ws_bytes, nv.ptr(st),
                                                    nv.stream(a.device)), "grouped_gemm_fp4_variable_k")
    nv.poll_status(out.device)
    return out


def grouped_gemm_fp4_variable_k_impl(a, b, a_scales, b_scales, group_lens, group_offs, out_dtype, granularity=None, num_cu=None,
                                     default_backend: int = 0):
    """C[g] = a[:, seg g] . b[:, seg g]^T over the 256-padded token segments: a [M, T/2], b [N, T/2] -> [G, M, N]."""
    return _variable_k(a, b, a_scales, b_scales, group_lens, group_offs, out_dtype, num_cu)


def grouped_gemm_fp4_variable_k_accum_impl(a, b, a_scales, b_scales, group_lens, group_offs, out, granularity=None, num_cu=None,
                                           default_backend: int = 0):
    return _variable_k(a, b, a_scales, b_scales, group_lens, group_offs, out.dtype, num_cu, out=out)
