"""Multi-threaded torch-CPU port of the path, used as the timed CPU baseline (test infrastructure).

The numpy oracle is the bit-level checker but runs on one core.  This module restates the same
arithmetic with torch CPU tensor ops (which use every host thread) so that a bounded sample of the
benchmark workload finishes in seconds.  tests/test_oracle_torch_port.py checks it against the
numpy oracle bit for bit.  Its fp32 -> fp8 step is torch's CPU cast, the same cast the reference's
own torch oracle uses (tests/pytorch/ref/quantization_ref.py:31-56).
"""
import torch

_FP8 = {"e4m3": (torch.float8_e4m3fn, 448.0, 3, 8), "e5m2": (torch.float8_e5m2, 57344.0, 2, 15)}


def mx_quantize_rows(x: torch.Tensor, fmt: str, use_2d_block: bool = False):
    """x [R, C] float32 with R % 32 == 0 (2-D mode) and C % 32 == 0 -> (q fp8 [R, C], scale uint8 [R, C/32]).
    Scale rule of csrc/kernels/quantization/quantization_mxfp8.cu:68-105, value rule :125-146."""
    dt, qmax, mbits, target = _FP8[fmt]
    R, C = x.shape
    blk = x.reshape(R, C // 32, 32)
    amax = blk.abs().amax(dim=2)
    if use_2d_block:
        amax = amax.reshape(R // 32, 32, C // 32).amax(dim=1, keepdim=True).expand(R // 32, 32, C // 32).reshape(R, C // 32)
    bits = amax.contiguous().view(torch.int32).to(torch.int64)
    e = (((bits + (1 << (22 - mbits))) >> 23) & 0x1FF) - 127 - target
    e = e.clamp(-127, 128)
    byte = (e + 127).to(torch.uint8)
    scale = ((e + 127).to(torch.int32) << 23).view(torch.float32)  # byte 0 -> 0.0f
    s = scale.unsqueeze(2)
    lim = qmax * s
    v = torch.minimum(torch.maximum(blk, -lim), lim) / s
    v = torch.where(s == 0, torch.zeros((), dtype=torch.float32), v)
    return v.reshape(R, C).to(dt), byte


def mx_dequantize_rows(q: torch.Tensor, byte: torch.Tensor) -> torch.Tensor:
    R, C = q.shape
    e = byte.to(torch.int32) - 127
    s = torch.ldexp(torch.ones_like(e, dtype=torch.float32), e)
    return (q.to(torch.float32).reshape(R, C // 32, 32) * s.unsqueeze(2)).reshape(R, C)


def mx_weight_prepare(w: torch.Tensor, fmt: str = "e4m3") -> torch.Tensor:
    """The weight half of the MX forward: dual (row + transposed col) quantization of w [N, K] with 2-D block scales;
    returns the dequantized row-wise copy the GEMM consumes (the col-wise copy is what backward would read)."""
    wf = w.float()
    w_row = mx_quantize_rows(wf, fmt, use_2d_block=True)
    _w_col = mx_quantize_rows(wf.t().contiguous(), fmt, use_2d_block=True)
    return mx_dequantize_rows(*w_row)


def mx_activation_forward(a: torch.Tensor, w_deq: torch.Tensor, fmt: str = "e4m3") -> torch.Tensor:
    """The activation half: dual MX quantization of a [M, K], then dequant(a_row) . w_deq^T in fp32, returned as bf16.
    Every part of it is linear in the number of activation rows."""
    af = a.float()
    a_row = mx_quantize_rows(af, fmt)
    _a_col = mx_quantize_rows(af.t().contiguous(), fmt)
    return (mx_dequantize_rows(*a_row) @ w_deq.t()).to(torch.bfloat16)


def mx_linear_forward(a: torch.Tensor, w: torch.Tensor, fmt: str = "e4m3") -> torch.Tensor:
    """The reference's MX forward (primus_turbo/pytorch/ops/gemm_fp8.py:558-654) on the CPU: dual (row +
    transposed col) MX quantization of a [M, K] and of w [N, K] (2-D block scales), then
    out = dequant(a_row) . dequant(w_row)^T accumulated in fp32, returned as bf16."""
    return mx_activation_forward(a, mx_weight_prepare(w, fmt), fmt)


def tensorwise_quantize(x: torch.Tensor, fmt: str):
    """Kernel arithmetic of csrc/include/primus_turbo/device/quant_utils.cuh:33-74 (true division)."""
    dt, qmax, _, _ = _FP8[fmt]
    xf = x.float()
    amax = xf.abs().amax().clamp(min=1e-12)
    scale = torch.tensor(qmax, dtype=torch.float32) / amax
    q = (xf * scale).clamp(-qmax, qmax).to(dt)
    return q, 1.0 / scale
