"""pt_quantize_fp8_colscale_noalloc: the column-scaled FP8 quantizer for callers that cannot allocate device
memory (a runtime whose arena already owns all of HBM, or code running where the driver's allocator may not be
called).  It keeps its scratch in an array built into the library, so it must give exactly the bytes and scales
of the workspace-taking entry point, call after call, although the built-in array still holds the previous
call's maxima when the next call starts.  Collected last on purpose: a failure here cannot hide other tests."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _both(x, fmt_dtype):
    from primus_turbo.pytorch.kernels import _native as nv
    B, M, N = x.shape
    lib = nv.lib()
    stream = nv.stream(x.device)
    q_ref = torch.empty_like(x, dtype=fmt_dtype)
    s_ref = torch.empty((B, 1, N), dtype=torch.float32, device=x.device)
    ws = torch.empty(B * N, dtype=torch.int32, device=x.device)
    nv.check(lib.pt_quantize_fp8_rowwise(nv.ptr(x), nv.src_code(x.dtype), B, M, N, 0, nv.fmt_code(fmt_dtype), nv.ptr(q_ref),
                                         nv.ptr(s_ref), None, nv.ptr(ws), ws.numel() * 4, stream), "pt_quantize_fp8_rowwise")
    q_new = torch.empty_like(x, dtype=fmt_dtype)
    s_new = torch.empty((B, 1, N), dtype=torch.float32, device=x.device)
    nv.check(lib.pt_quantize_fp8_colscale_noalloc(nv.ptr(x), nv.src_code(x.dtype), B, M, N, nv.fmt_code(fmt_dtype),
                                                  nv.ptr(q_new), nv.ptr(s_new), stream), "pt_quantize_fp8_colscale_noalloc")
    torch.cuda.synchronize()
    return q_ref, s_ref, q_new, s_new


def test_matches_workspace_entry_point_on_two_calls_in_a_row():
    g = torch.Generator().manual_seed(99)
    # first call: large values; second call: small ones in the same columns, so maxima left over from the first
    # call would give wrong (too small) scales if the array were not cleared
    x1 = (torch.randn(2, 300, 520, generator=g) * 40).to(torch.bfloat16).cuda()
    x2 = (torch.randn(2, 300, 520, generator=g) * 1e-3).to(torch.bfloat16).cuda()
    for x in (x1, x2):
        q_ref, s_ref, q_new, s_new = _both(x, torch.float8_e4m3fn)
        assert torch.equal(s_new, s_ref)                                  # scales: bit-exact, as in the other quantizer tests
        assert torch.equal(q_new.view(torch.uint8), q_ref.view(torch.uint8))  # bytes: bit-exact
    # a third shape and the other format, still right after the calls above
    x3 = torch.randn(1, 77, 4096, generator=g).to(torch.float32).cuda()
    q_ref, s_ref, q_new, s_new = _both(x3, torch.float8_e5m2)
    assert torch.equal(s_new, s_ref) and torch.equal(q_new.view(torch.uint8), q_ref.view(torch.uint8))


def test_refuses_more_columns_than_the_built_in_scratch():
    from primus_turbo.pytorch.kernels import _native as nv
    x = torch.zeros(1, 2, 65536 + 8, dtype=torch.bfloat16, device="cuda")
    q = torch.empty_like(x, dtype=torch.float8_e4m3fn)
    s = torch.empty((1, 1, x.shape[2]), dtype=torch.float32, device="cuda")
    rc = nv.lib().pt_quantize_fp8_colscale_noalloc(nv.ptr(x), nv.src_code(x.dtype), 1, 2, x.shape[2], nv.fmt_code(q.dtype),
                                                   nv.ptr(q), nv.ptr(s), nv.stream(x.device))
    assert rc == -1
    assert b"exceed the built-in scratch" in nv.lib().pt_last_error()
