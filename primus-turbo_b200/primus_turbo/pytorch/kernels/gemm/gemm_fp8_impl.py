"""FP8 / MXFP8 dense GEMM over the C ABI.

Same call shape as primus_turbo::gemm_fp8_impl / gemm_fp8_accum_impl of the reference
(primus_turbo/pytorch/kernels/gemm/gemm_fp8_impl.py:518-593).  The CUDA kernel computes
C = A . B^T with both operands K-major; the other (trans_a, trans_b, trans_c) combinations are
mapped onto it by swapping the operands (trans_c) or by transposing the FP8 bytes first, which is
what the reference does for its NT-only back ends (primus_turbo/pytorch/ops/gemm_fp8.py:44-50).
"""
import torch

from ...core.low_precision import ScalingGranularity
from .. import _native as nv
from ..quantization.quantization_impl import transpose_2d

_GRAN = {ScalingGranularity.TENSORWISE: nv.PT_TENSORWISE, ScalingGranularity.ROWWISE: nv.PT_ROWWISE,
         ScalingGranularity.BLOCKWISE: nv.PT_BLOCKWISE, ScalingGranularity.MX_BLOCKWISE: nv.PT_MX_BLOCKWISE}


def _as_gran(granularity):
    return granularity if isinstance(granularity, ScalingGranularity) else ScalingGranularity(int(granularity))


def _k_major(x, trans):
    """Returns x laid out [rows, K] with K a multiple of 16 bytes (a TMA row pitch requirement): x itself when
    it already is, else the transposed bytes; a ragged contraction length is zero padded."""
    if not trans:
        x = x.contiguous()
        K = x.shape[1]
        if K % 16 == 0:
            return x
        y = torch.zeros((x.shape[0], (K + 15) // 16 * 16), dtype=torch.uint8, device=x.device)
        y[:, :K] = x.view(torch.uint8)
        return y.view(x.dtype)
    K = x.shape[0]
    if K % 16 == 0:
        return transpose_2d(x)
    y = torch.zeros((x.shape[1], (K + 15) // 16 * 16), dtype=torch.uint8, device=x.device)
    y[:, :K] = x.view(torch.uint8).t()
    return y.view(x.dtype)


def _block_scale_desc(scale, rows, kc, source_transposed):
    """(shift, row_stride, kb_stride) that reads `scale` for a K-major operand of `rows` rows and contraction
    length `kc`, given whether the operand's source tensor was stored contraction-major (transposed)."""
    kb = (kc + 127) // 128
    rb = (rows + 127) // 128
    s0, s1 = scale.shape
    if not source_transposed:           # source [rows, kc]
        assert s1 == kb, f"blockwise scale shape {tuple(scale.shape)} does not match contraction {kc}"
        if s0 == rows:
            return 0, s1, 1
        assert s0 == rb, f"blockwise scale shape {tuple(scale.shape)} does not match {rows} rows"
        return 7, s1, 1
    assert s0 == kb, f"blockwise scale shape {tuple(scale.shape)} does not match contraction {kc}"
    if s1 == rows:                      # source [kc, rows], one scale per (K block, row)
        return 0, 1, s1
    assert s1 == rb, f"blockwise scale shape {tuple(scale.shape)} does not match {rows} rows"
    return 7, 1, s1


def _bw_operand(x, trans_to_kmajor):
    """(tensor, mn_major, mem_rows, mem_cols): a K-major operand is used as stored; one stored contraction-major is
    used as stored too (MN-major) when its row pitch allows, else transposed into a zero-padded K-major copy."""
    x = x.contiguous()
    if not trans_to_kmajor:
        xk = _k_major(x, False)
        return xk, 0, xk.shape[0], xk.shape[1]
    if x.shape[1] % 16 == 0:
        return x, 1, x.shape[0], x.shape[1]
    xk = _k_major(x, True)
    return xk, 0, xk.shape[0], xk.shape[1]


def _launch_blockwise(a_op, a_desc, a_s, b_op, b_desc, b_s, out, beta, M, N, kc):
    a_t, a_mn, a_r, a_c = a_op
    b_t, b_mn, b_r, b_c = b_op
    K = kc if (a_mn and b_mn) else (a_t.shape[1] if not a_mn else (b_t.shape[1] if not b_mn else kc))
    if not (a_mn and b_mn):
        # a K-major operand may carry zero padding up to a multiple of 16; the other side must agree on K
        K = max(K, kc)
    st = nv.status_word(out.device)
    with nv.on_device(out.device):
        nv.check(nv.lib().pt_grouped_gemm_fp8_blockwise(
            nv.ptr(a_t), nv.fmt_code(a_t.dtype), a_mn, a_r, a_c, nv.ptr(a_s), *a_desc,
            nv.ptr(b_t), nv.fmt_code(b_t.dtype), b_mn, b_r, b_c, nv.ptr(b_s), *b_desc, 0,
            nv.ptr(out), nv.src_code(out.dtype), M, N, K, None, None, None, 1, float(beta), 0, nv.ptr(st),
            nv.stream(out.device)), "gemm_fp8_blockwise")
    nv.poll_status(out.device)
    return out


def _launch(a_km, a_s, b_km, b_s, out, gran, beta, block_n=0):
    M, K = a_km.shape
    N = b_km.shape[0]
    assert b_km.shape[1] == K, f"contraction mismatch: {a_km.shape} vs {b_km.shape}"
    st = nv.status_word(out.device)
    ws_bytes = nv.lib().pt_gemm_fp8_workspace_bytes(_GRAN[gran], M, N, K, 1, 0, block_n)
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device=out.device) if ws_bytes else None
    with nv.on_device(out.device):
        nv.check(nv.lib().pt_gemm_fp8(nv.ptr(a_km), nv.ptr(a_s), nv.fmt_code(a_km.dtype), nv.ptr(b_km), nv.ptr(b_s),
                                       nv.fmt_code(b_km.dtype), nv.ptr(out), nv.src_code(out.dtype), _GRAN[gran], M, N, K,
                                       float(beta), block_n, nv.ptr(ws), ws_bytes, nv.ptr(st), nv.stream(out.device)),
                 "gemm_fp8")
    nv.poll_status(out.device)
    return out


def _launch_mn(a_t, a_mn, a_s, b_t, b_mn, b_s, out, gran, beta, M, N, K):
    """Tensorwise / rowwise with at least one operand read contraction-major in place."""
    st = nv.status_word(out.device)
    with nv.on_device(out.device):
        nv.check(nv.lib().pt_gemm_fp8_mn(nv.ptr(a_t), nv.ptr(a_s), nv.fmt_code(a_t.dtype), a_mn, nv.ptr(b_t), nv.ptr(b_s),
                                          nv.fmt_code(b_t.dtype), b_mn, nv.ptr(out), nv.src_code(out.dtype), _GRAN[gran], M, N, K,
                                          float(beta), nv.ptr(st), nv.stream(out.device)), "gemm_fp8_mn")
    nv.poll_status(out.device)
    return out


def _gemm(a, a_scale_inv, trans_a, b, b_scale_inv, trans_b, out_dtype, trans_c, granularity, out=None, block_n=0,
          accumulate=True):
    """`out` given: accumulate into it (beta = 1), or overwrite it when accumulate is False."""
    nv.require_cuda(a, b, a_scale_inv, b_scale_inv)
    assert a.dim() == 2 and b.dim() == 2, "Only 2D tensors are supported"
    gran = _as_gran(granularity)
    if gran == ScalingGranularity.BLOCKWISE:
        M = a.shape[1] if trans_a else a.shape[0]
        N = b.shape[0] if trans_b else b.shape[1]
        kc = a.shape[0] if trans_a else a.shape[1]
        a_s, b_s = a_scale_inv.to(torch.float32).contiguous(), b_scale_inv.to(torch.float32).contiguous()
        a_desc = _block_scale_desc(a_s, M, kc, trans_a)
        b_desc = _block_scale_desc(b_s, N, kc, not trans_b)
        a_op, b_op = _bw_operand(a, trans_a), _bw_operand(b, not trans_b)
        if (a_op[1] == 0) != (b_op[1] == 0) and kc % 16 != 0:
            # a ragged contraction cannot mix a padded K-major copy with an MN-major operand read in place
            a_op = (_k_major(a, trans_a), 0) + tuple(_k_major(a, trans_a).shape)
            b_op = (_k_major(b, not trans_b), 0) + tuple(_k_major(b, not trans_b).shape)
        beta = 0.0
        if out is not None:
            beta = 1.0 if accumulate else 0.0
            assert out.is_contiguous() and tuple(out.shape) == ((N, M) if trans_c else (M, N))
        else:
            out = torch.empty((N, M) if trans_c else (M, N), dtype=out_dtype, device=a.device)
        if trans_c:
            return _launch_blockwise(b_op, b_desc, b_s, a_op, a_desc, a_s, out, beta, N, M, kc)
        return _launch_blockwise(a_op, a_desc, a_s, b_op, b_desc, b_s, out, beta, M, N, kc)
    if gran == ScalingGranularity.MX_BLOCKWISE:
        assert not trans_a and trans_b, "MX GEMM takes K-major operands only (trans_a=False, trans_b=True)"
    a_s = a_scale_inv.contiguous()
    b_s = b_scale_inv.contiguous()
    if gran in (ScalingGranularity.TENSORWISE, ScalingGranularity.ROWWISE) and block_n == 0 and (trans_a or not trans_b):
        # an operand stored contraction-major ([K, rows]) is read in place (MN-major) when its row pitch allows; the
        # transposed copy below remains for ragged shapes
        M = a.shape[1] if trans_a else a.shape[0]
        N = b.shape[0] if trans_b else b.shape[1]
        kc = a.shape[0] if trans_a else a.shape[1]
        a_mn, b_mn = int(trans_a), int(not trans_b)
        ok = (not a_mn or M % 16 == 0) and (not b_mn or N % 16 == 0) and (kc % 16 == 0 or (a_mn and b_mn))
        a_c, b_c = a.contiguous(), b.contiguous()
        if ok and a_c.data_ptr() % 16 == 0 and b_c.data_ptr() % 16 == 0:
            a_f, b_f = a_s.to(torch.float32).reshape(-1), b_s.to(torch.float32).reshape(-1)
            if gran == ScalingGranularity.ROWWISE:
                assert a_f.numel() == M and b_f.numel() == N, "rowwise scales must match M and N"
            beta = 0.0
            if out is not None:
                beta = 1.0 if accumulate else 0.0
                assert out.is_contiguous() and tuple(out.shape) == ((N, M) if trans_c else (M, N))
            else:
                out = torch.empty((N, M) if trans_c else (M, N), dtype=out_dtype, device=a.device)
            if trans_c:
                return _launch_mn(b_c, b_mn, b_f, a_c, a_mn, a_f, out, gran, beta, N, M, kc)
            return _launch_mn(a_c, a_mn, a_f, b_c, b_mn, b_f, out, gran, beta, M, N, kc)
    a_km = _k_major(a, trans_a)            # [M, K]
    b_km = _k_major(b, not trans_b)        # [N, K]
    if gran in (ScalingGranularity.TENSORWISE, ScalingGranularity.ROWWISE):
        a_s, b_s = a_s.to(torch.float32).reshape(-1), b_s.to(torch.float32).reshape(-1)
        if gran == ScalingGranularity.ROWWISE:
            assert a_s.numel() == a_km.shape[0] and b_s.numel() == b_km.shape[0], "rowwise scales must match M and N"
    M, N = a_km.shape[0], b_km.shape[0]
    beta = 0.0
    if out is not None:
        beta = 1.0 if accumulate else 0.0
        assert out.is_contiguous() and tuple(out.shape) == ((N, M) if trans_c else (M, N))
    else:
        out = torch.empty((N, M) if trans_c else (M, N), dtype=out_dtype, device=a.device)
    if trans_c:
        return _launch(b_km, b_s, a_km, a_s, out, gran, beta, block_n)
    return _launch(a_km, a_s, b_km, b_s, out, gran, beta, block_n)


def gemm_fp8_impl(a, a_scale_inv, trans_a, b, b_scale_inv, trans_b, out_dtype, trans_c, granularity,
                  default_backend=0, block_n=0, out=None):
    """C = op(A) . op(B) (optionally transposed). `default_backend` is accepted and ignored: there is one back end.
    `out` (contiguous, result shape and dtype) is written instead of a fresh tensor: a caller that owns a larger buffer
    (a gather buffer, a preallocated activation) passes the slot the result belongs in."""
    return _gemm(a, a_scale_inv, trans_a, b, b_scale_inv, trans_b, out_dtype if out is None else out.dtype, trans_c,
                 granularity, out, block_n, accumulate=False)


def gemm_fp8_accum_impl(a, a_scale_inv, trans_a, b, b_scale_inv, trans_b, out, trans_c, granularity, default_backend=0):
    """out += op(A) . op(B); `out` is modified in place and returned."""
    return _gemm(a, a_scale_inv, trans_a, b, b_scale_inv, trans_b, out.dtype, trans_c, granularity, out)
