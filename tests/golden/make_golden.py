"""Generate the golden fixtures in this directory from the REFERENCE's own code.

Run in the build container only (the reference tree is not present on a GPU
box):   python tests/golden/make_golden.py /path/to/reference

Two reference code paths run on a CPU and are used here:

* tests/pytorch/ref/quantization_ref.py -- the reference's pure-torch
  tensorwise / rowwise quantizers (its own test oracle).  It imports one enum
  from the reference package, which cannot be imported without a GPU, so a
  two-member stand-in enum is injected.
* primus_turbo/triton/quantization/quant_blockwise.py -- the reference's Triton
  blockwise kernels, executed by Triton's CPU interpreter (TRITON_INTERPRET=1).
  The interpreter's own float32 -> fp8 cast drops the carry when the mantissa
  rounds up into the next binade (126.2 became 64 instead of 128), so the
  kernels are given float32 output buffers -- their final `.to(element_ty)` is
  then the identity and they deliver the scaled, clamped float32 values -- and
  the last step, the cast to fp8, is done by torch's CPU cast, the same cast
  the reference's torch oracle uses.

The torch reference forms `fp8_max / amax` as reciprocal(amax) * fp8_max (that is how
torch evaluates scalar / tensor), one rounding more than the kernels' true division, so its
scale can sit one ulp from the kernel's.  The fixture therefore also stores the reference's
`scale`, and the oracle's multiply / clamp / round-to-nearest-even cast is pinned bit for bit
given that scale, while the scale itself is pinned to one ulp.  The Triton blockwise kernels
divide truly and pin the scale formula bit for bit.

The fixtures hold inputs (as uint16 bf16 bit patterns or float32) and the
reference outputs (raw fp8 bytes, float32 scales) in one .npz per family.
"""
import enum
import importlib.util
import os
import sys
import types

os.environ["TRITON_INTERPRET"] = "1"

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
REF = sys.argv[1] if len(sys.argv) > 1 else "/root/reference"


def _load(path, name):
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def _stub_low_precision():
    class ScalingGranularity(enum.Enum):
        TENSORWISE = enum.auto()
        ROWWISE = enum.auto()

    names = ["primus_turbo", "primus_turbo.pytorch", "primus_turbo.pytorch.core",
             "primus_turbo.pytorch.core.low_precision"]
    for n in names:
        sys.modules.setdefault(n, types.ModuleType(n))
    sys.modules[names[-1]].ScalingGranularity = ScalingGranularity
    return ScalingGranularity


def bf16_bits(t: torch.Tensor) -> np.ndarray:
    return t.view(torch.int16).numpy().view(np.uint16).copy()


def u8(t: torch.Tensor) -> np.ndarray:
    return t.view(torch.uint8).numpy().copy()


def make_inputs(gen, shape, kind):
    x = torch.randn(*shape, generator=gen)
    if kind == "outlier":
        mask = torch.rand(*shape, generator=gen) < 0.01
        x = torch.where(mask, x * 50, x)
    elif kind == "small":
        x = x * 1e-3
    elif kind == "zeros_mixed":
        x[: max(1, shape[0] // 3)] = 0
    return x


def tensor_row(out):
    SG = _stub_low_precision()
    qr = _load(os.path.join(REF, "tests/pytorch/ref/quantization_ref.py"), "quantization_ref")
    gen = torch.Generator().manual_seed(42)
    cases = []
    for dt_name, dt in (("e4m3", torch.float8_e4m3fn), ("e5m2", torch.float8_e5m2)):
        for shape, kind in (((1, 17), "plain"), ((33, 128), "outlier"), ((64, 257), "small"), ((5, 2881), "plain")):
            # tensorwise: fp32 input (the torch reference multiplies bf16 inputs in bf16,
            # the kernels in fp32; for fp32 inputs the two coincide bit for bit)
            x = make_inputs(gen, shape, kind)
            q, sc, sinv = qr.quantize_fp8_ref(x, dt, SG.TENSORWISE)
            cases.append(dict(kind="tensorwise", fmt=dt_name, x=x.numpy(), q=u8(q), s=sinv.numpy(), scale=sc.numpy()))
            for axis in (-1, -2):
                xb = make_inputs(gen, shape, kind).to(torch.bfloat16)
                q, sc, sinv = qr.quantize_fp8_ref(xb, dt, SG.ROWWISE, axis=axis)
                cases.append(dict(kind="rowwise", fmt=dt_name, axis=axis, x_bf16=bf16_bits(xb), q=u8(q), s=sinv.numpy(),
                                  scale=sc.numpy()))
    flat = {}
    for i, c in enumerate(cases):
        for k, v in c.items():
            flat[f"c{i}_{k}"] = np.asarray(v)
    flat["n"] = np.asarray(len(cases))
    np.savez_compressed(os.path.join(out, "tensor_row.npz"), **flat)
    print("tensor_row.npz", len(cases), "cases")


def blockwise(out):
    qb = _load(os.path.join(REF, "primus_turbo/triton/quantization/quant_blockwise.py"), "quant_blockwise")
    gen = torch.Generator().manual_seed(43)
    B = 128
    cdiv = lambda a, b: (a + b - 1) // b
    flat, n = {}, 0
    for dt_name, dt, fmax in (("e4m3", torch.float8_e4m3fn, 448.0), ("e5m2", torch.float8_e5m2, 57344.0)):
        for (M, N), kind in (((136, 256), "plain"), ((128, 130), "outlier"), ((257, 128), "zeros_mixed")):
            x = make_inputs(gen, (M, N), kind).to(torch.bfloat16)
            grid = (cdiv(M, B), cdiv(N, B))
            # 1-D, both axes
            for axis in (1, 0):
                q = torch.zeros(M, N, dtype=torch.float32)
                s = torch.zeros((M, cdiv(N, B)) if axis == 1 else (cdiv(M, B), N), dtype=torch.float32)
                qb.quant_fp8_blockwise_kernel[grid](x, q, s, M, N, B, fmax, axis)
                flat.update({f"c{n}_kind": np.asarray("blockwise"), f"c{n}_fmt": np.asarray(dt_name),
                             f"c{n}_axis": np.asarray(axis), f"c{n}_x_bf16": bf16_bits(x),
                             f"c{n}_q": u8(q.to(dt)), f"c{n}_s": s.numpy().copy()})
                n += 1
            # dual
            qr_, qc_ = torch.zeros(M, N, dtype=torch.float32), torch.zeros(M, N, dtype=torch.float32)
            sr_, sc_ = torch.zeros(M, cdiv(N, B)), torch.zeros(cdiv(M, B), N)
            qb.quant_fp8_blockwise_dual_kernel[grid](x, qr_, sr_, qc_, sc_, M, N, B, fmax)
            flat.update({f"c{n}_kind": np.asarray("dual"), f"c{n}_fmt": np.asarray(dt_name),
                         f"c{n}_x_bf16": bf16_bits(x), f"c{n}_q": u8(qr_.to(dt)), f"c{n}_s": sr_.numpy().copy(),
                         f"c{n}_q2": u8(qc_.to(dt)), f"c{n}_s2": sc_.numpy().copy()})
            n += 1
            # 128x128 weight tiles, batched
            w = torch.stack([x, make_inputs(gen, (M, N), "small").to(torch.bfloat16)])
            qw = torch.zeros(2, M, N, dtype=torch.float32)
            sw = torch.zeros(2, cdiv(M, B), cdiv(N, B))
            qb.quant_fp8_blockwise_for_weight_kernel[(2,) + grid](w, qw, sw, M, N, B, fmax)
            flat.update({f"c{n}_kind": np.asarray("weight"), f"c{n}_fmt": np.asarray(dt_name),
                         f"c{n}_x_bf16": bf16_bits(w), f"c{n}_q": u8(qw.to(dt)), f"c{n}_s": sw.numpy().copy()})
            n += 1
        # segment-M row + col (grouped), with an empty group and ragged lengths
        for lens in ([100, 0, 128, 29], [1, 300]):
            lens_t = torch.tensor(lens, dtype=torch.int64)
            M, N, G = int(lens_t.sum()), 256, len(lens)
            x = make_inputs(gen, (M, N), "outlier").to(torch.bfloat16)
            offs = torch.zeros(G + 1, dtype=torch.int64)
            offs[1:] = torch.cumsum(lens_t, 0)
            plens = (lens_t + B - 1) // B * B
            poffs = torch.zeros(G + 1, dtype=torch.int64)
            poffs[1:] = torch.cumsum(plens, 0)
            m_alloc = M + G * B
            q_row = torch.zeros(M, N, dtype=torch.float32)
            q_col = torch.zeros(m_alloc, N, dtype=torch.float32)
            s_row = torch.zeros(cdiv(N, B), M)
            s_col = torch.zeros(m_alloc // B, N)
            qb.quant_fp8_blockwise_segment_m_row_col_kernel[(cdiv(m_alloc, B), cdiv(N, B))](
                x, q_row, q_col, s_row, s_col, offs, poffs, M, N, G, B, fmax)
            flat.update({f"c{n}_kind": np.asarray("segment_m"), f"c{n}_fmt": np.asarray(dt_name),
                         f"c{n}_lens": np.asarray(lens, dtype=np.int64), f"c{n}_x_bf16": bf16_bits(x),
                         f"c{n}_q": u8(q_row.to(dt)), f"c{n}_s": s_row.numpy().copy(),
                         f"c{n}_q2": u8(q_col.to(dt)), f"c{n}_s2": s_col.numpy().copy()})
            n += 1
    flat["n"] = np.asarray(n)
    np.savez_compressed(os.path.join(out, "blockwise.npz"), **flat)
    print("blockwise.npz", n, "cases")


if __name__ == "__main__":
    tensor_row(HERE)
    blockwise(HERE)
