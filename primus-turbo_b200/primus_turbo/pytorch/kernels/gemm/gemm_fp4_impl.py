"""MXFP4 dense GEMM over the C ABI (primus_turbo::gemm_fp4_impl / gemm_fp4_accum_impl of the reference,
primus_turbo/pytorch/kernels/gemm/gemm_fp4_impl.py:340-441).  NT only: both operands packed e2m1, K-major."""
import torch

from .. import _native as nv


def _gemm_fp4(a, a_scale_inv, trans_a, b, b_scale_inv, trans_b, out_dtype, trans_c, out=None):
    nv.require_cuda(a, b, a_scale_inv, b_scale_inv)
    assert not trans_a and trans_b, "MXFP4 GEMM takes K-major operands only (trans_a=False, trans_b=True)"
    assert a.dtype == torch.float4_e2m1fn_x2 and b.dtype == torch.float4_e2m1fn_x2
    a, b = a.contiguous(), b.contiguous()
    a_s, b_s = a_scale_inv.contiguous(), b_scale_inv.contiguous()
    if trans_c:
        a, a_s, b, b_s = b, b_s, a, a_s
    M, N = a.shape[0], b.shape[0]
    K = a.view(torch.uint8).shape[1] * 2
    assert b.view(torch.uint8).shape[1] * 2 == K, "contraction mismatch"
    beta = 0.0
    if out is None:
        out = torch.empty((M, N), dtype=out_dtype, device=a.device)
    else:
        beta = 1.0
        assert tuple(out.shape) == (M, N) and out.is_contiguous()
    lib = nv.lib()
    ws_bytes = lib.pt_gemm_fp4_workspace_bytes(M, N, K, 1, 0, 0)
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device=a.device)
    st = nv.status_word(a.device)
    with nv.on_device(a.device):
        nv.check(lib.pt_gemm_fp4(nv.ptr(a), nv.ptr(a_s), nv.ptr(b), nv.ptr(b_s), nv.ptr(out), nv.src_code(out.dtype), M, N, K, beta, 0,
                                 nv.ptr(ws), ws_bytes, nv.ptr(st), nv.stream(a.device)), "gemm_fp4")
    nv.poll_status(out.device)
    return out


def gemm_fp4_impl(a, a_scale_inv, trans_a, b, b_scale_inv, trans_b, out_dtype, trans_c, granularity=None, default_backend=0,
                  preshuffled=False):
    assert not preshuffled, "pre-shuffled operands are not provided on B200"
    return _gemm_fp4(a, a_scale_inv, trans_a, b, b_scale_inv, trans_b, out_dtype, trans_c)


def gemm_fp4_accum_impl(a, a_scale_inv, trans_a, b, b_scale_inv, trans_b, out, trans_c, granularity=None, default_backend=0,
                        preshuffled=False):
    assert not preshuffled, "pre-shuffled operands are not provided on B200"
    return _gemm_fp4(a, a_scale_inv, trans_a, b, b_scale_inv, trans_b, out.dtype, trans_c, out=out)
