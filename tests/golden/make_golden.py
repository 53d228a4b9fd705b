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

* MX (mx.npz): three more pieces of the reference run here.  (1) `compute_tile_scale`
  (csrc/kernels/quantization/quantization_mxfp8.cu:68-105, quantization_mxfp4.cu:149-181) and
  `e8m0_to_scale` (csrc/include/primus_turbo/device/utils.cuh:124-126), compiled on the host by
  oracle/build_ref.py: ue8m0 bytes and native scales for every non-negative bf16 bit pattern and
  4096 float32 patterns as block amax, for e4m3 / e5m2 / e2m1, and the decode of all 256 scale
  bytes.  (2) `_dequant_mxfp8` (tests/pytorch/modules/test_mega_moe_mxfp8.py:57-62), a torch
  dequantizer, run on random code / scale bytes.  (3) `mxfp8_padded_ref` / `mxfp4_padded_ref`
  (tests/pytorch/ops/test_quantization.py:288-340), which fix the zero-padded layouts of the row-wise,
  column-wise and batched outputs.  The two test helpers are taken out of their files by name (the files
  import the reference package, which cannot be imported without a GPU) and executed unchanged.
  What stays unpinned is the final fp32 -> fp8 / fp4 rounding of an AMD convert instruction.

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


def _functions_from(path, names):
    """Executes the named top-level functions of a reference test file (and nothing else of it) in a namespace that
    provides torch; returns the namespace."""
    import ast
    src = open(path).read()
    tree = ast.parse(src)
    keep = [n for n in tree.body if isinstance(n, ast.FunctionDef) and n.name in names]
    assert len(keep) == len(names), f"{path}: expected functions {names}"
    ns = {"torch": torch, "_MXFP8_BLOCK": 32}
    exec(compile(ast.Module(body=keep, type_ignores=[]), path, "exec"), ns)
    return ns


def mx(out):
    sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
    from oracle import build_ref
    build_ref.build(REF)
    lib = build_ref.load()
    flat = {}
    # (1) scale rule: every non-negative bf16 pattern (incl. inf / NaN patterns) + float32 patterns with low bits set
    rng = np.random.default_rng(44)
    amax_bits = np.concatenate([np.arange(0x8000, dtype=np.uint32) << 16,
                                rng.integers(0, 0x7F800000, size=4096, dtype=np.uint32)])
    flat["scale_amax_bits"] = amax_bits
    for fmt in ("e4m3", "e5m2", "e2m1"):
        byte, native = build_ref.tile_scale(lib, fmt, amax_bits.view(np.float32))
        flat[f"scale_byte_{fmt}"] = byte
        flat[f"scale_native_bits_{fmt}"] = native.view(np.uint32)
    dec = np.empty(256, dtype=np.float32)
    allb = np.arange(256, dtype=np.uint8)
    lib.ref_e8m0_to_scale(allb.ctypes.data, 256, dec.ctypes.data)
    flat["e8m0_decode_bits"] = dec.view(np.uint32)
    # (2) the reference's torch dequantizer on random codes and scale bytes (NaN codes excluded: NaN != NaN)
    deq = _functions_from(os.path.join(REF, "tests/pytorch/modules/test_mega_moe_mxfp8.py"), ["_dequant_mxfp8"])["_dequant_mxfp8"]
    for fmt, dt in (("e4m3", torch.float8_e4m3fn), ("e5m2", torch.float8_e5m2)):
        codes = rng.integers(0, 256, size=(16, 256), dtype=np.uint8)
        if fmt == "e4m3":
            codes[(codes & 0x7F) == 0x7F] = 0x3A
        else:
            codes[(codes & 0x7C) == 0x7C] = 0x3A
        sbytes = rng.integers(90, 160, size=(16, 8), dtype=np.uint8)
        y = deq(torch.from_numpy(codes).view(dt), torch.from_numpy(sbytes))
        flat[f"deq_codes_{fmt}"], flat[f"deq_scales_{fmt}"], flat[f"deq_out_{fmt}"] = codes, sbytes, y.numpy().copy()
    # (3) padded layouts
    pads = _functions_from(os.path.join(REF, "tests/pytorch/ops/test_quantization.py"), ["padding_size", "mxfp8_padded_ref", "mxfp4_padded_ref"])
    gen = torch.Generator().manual_seed(45)
    n = 0
    for name in ("mxfp8_padded_ref", "mxfp4_padded_ref"):
        for shape, axis in (((33, 64), 0), ((33, 64), 1), ((130, 96), 0), ((130, 96), 1), ((2, 40, 64), 1), ((2, 40, 64), 2)):
            x = torch.randn(*shape, generator=gen).to(torch.bfloat16)
            ref = pads[name](x, axis, 128, torch.bfloat16)
            flat.update({f"pad{n}_fn": np.asarray(name), f"pad{n}_axis": np.asarray(axis), f"pad{n}_x_bf16": bf16_bits(x),
                         f"pad{n}_ref_bf16": bf16_bits(ref.contiguous())})
            n += 1
    flat["n_pad"] = np.asarray(n)
    np.savez_compressed(os.path.join(out, "mx.npz"), **flat)
    print("mx.npz", n, "padded-layout cases,", amax_bits.size, "amax patterns x 3 formats")


if __name__ == "__main__":
    tensor_row(HERE)
    blockwise(HERE)
    mx(HERE)
