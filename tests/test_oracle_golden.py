"""The CPU oracle against golden vectors produced by the reference's own code
(tests/golden/make_golden.py): pure-torch tensorwise/rowwise reference and the
Triton blockwise kernels run under the Triton CPU interpreter."""
import os

import numpy as np
import pytest

from oracle import quant as oq

GOLD = os.path.join(os.path.dirname(__file__), "golden")


def bf16_to_f32(bits):
    return (bits.astype(np.uint32) << 16).view(np.float32)


def _cases(name):
    z = np.load(os.path.join(GOLD, name))
    out = []
    for i in range(int(z["n"])):
        pre = f"c{i}_"
        out.append({k[len(pre):]: z[k] for k in z.files if k.startswith(pre)})
    return out


@pytest.mark.parametrize("case", _cases("tensor_row.npz"), ids=lambda c: f"{c['kind']}-{c['fmt']}-{c['q'].shape}")
def test_tensor_row(case):
    fmt = str(case["fmt"])
    if str(case["kind"]) == "tensorwise":
        q, s = oq.quantize_fp8_tensorwise(case["x"], fmt)
    else:
        q, s = oq.quantize_fp8_rowwise(bf16_to_f32(case["x_bf16"]), fmt, int(case["axis"]))
    # The torch reference evaluates fp8_max / amax as reciprocal * fp8_max (one extra rounding);
    # the kernels and the oracle divide.  scale is then within one ulp and scale_inv = 1/scale within
    # two.  Cast: bit-exact given the scale.
    assert s.shape == case["s"].shape
    ulp = np.abs(s.view(np.int32).astype(np.int64) - case["s"].view(np.int32).astype(np.int64))
    assert ulp.max() <= 2
    x = case["x"] if str(case["kind"]) == "tensorwise" else bf16_to_f32(case["x_bf16"])
    q_given = oq._quant_clamp_encode(x, case["scale"], fmt)
    assert np.array_equal(q_given, case["q"])
    # with its own scale the oracle may differ only where the scale differs
    amax = np.max(np.abs(x)) if str(case["kind"]) == "tensorwise" else np.max(np.abs(x), axis=int(case["axis"]), keepdims=True)
    own_scale, _ = oq._scale_from_amax(amax, fmt, 1e-12)
    same = np.broadcast_to(own_scale == case["scale"], q.shape)
    assert np.array_equal(q[same], case["q"][same])


@pytest.mark.parametrize("case", _cases("blockwise.npz"), ids=lambda c: f"{c['kind']}-{c['fmt']}-{c['q'].shape}")
def test_blockwise(case):
    fmt, kind = str(case["fmt"]), str(case["kind"])
    x = bf16_to_f32(case["x_bf16"])
    if kind == "blockwise":
        q, s = oq.quantize_fp8_blockwise(x, fmt, int(case["axis"]))
        got = [(q, case["q"]), (s, case["s"])]
    elif kind == "dual":
        qr, sr, qc, sc = oq.quantize_fp8_blockwise_dual(x, fmt)
        got = [(qr, case["q"]), (sr, case["s"]), (qc, case["q2"]), (sc, case["s2"])]
    elif kind == "weight":
        q, s = oq.quantize_fp8_blockwise_weight(x, fmt)
        got = [(q, case["q"]), (s, case["s"])]
    else:
        lens = case["lens"]
        q_row, q_col, s_row, s_col, plens, poffs = oq.quantize_fp8_blockwise_segment_m(x, fmt, lens)
        mp = int(poffs[-1])
        got = [(q_row, case["q"]), (s_row, case["s"]), (q_col[:mp], case["q2"][:mp]),
               (s_col[:mp // 128], case["s2"][:mp // 128])]
    for a, b in got:
        if a.dtype == np.float32:
            assert np.array_equal(a.view(np.uint32), b.view(np.uint32))
        else:
            assert np.array_equal(a, b)


# ------------------------------------------------------------------------------------------------ MX
def _mx():
    return np.load(os.path.join(GOLD, "mx.npz"))


@pytest.mark.parametrize("fmt", ["e4m3", "e5m2", "e2m1"])
def test_mx_scale_rule_against_the_reference_function(fmt):
    """ue8m0 byte and native scale for 32768 bf16 and 4096 float32 amax patterns: the reference's compute_tile_scale
    compiled on the host (oracle/build_ref.py)."""
    from oracle.codecs import mx_scale_from_amax
    z = _mx()
    amax = z["scale_amax_bits"].view(np.float32)
    byte, native = mx_scale_from_amax(amax, fmt)
    assert np.array_equal(byte, z[f"scale_byte_{fmt}"])
    assert np.array_equal(native.view(np.uint32), z[f"scale_native_bits_{fmt}"])


def test_mx_scale_rule_against_the_compiled_reference_when_present():
    """The same comparison on fresh random patterns, straight against oracle/_ref (built where the reference tree is
    available; skipped elsewhere)."""
    from oracle import build_ref
    from oracle.codecs import mx_scale_from_amax
    lib = build_ref.load()
    if lib is None:
        pytest.skip("oracle/_ref is not built here")
    bits = np.random.default_rng(7).integers(0, 0x7F800001, size=200000, dtype=np.uint32)
    for fmt in ("e4m3", "e5m2", "e2m1"):
        b_ref, n_ref = build_ref.tile_scale(lib, fmt, bits.view(np.float32))
        b, n = mx_scale_from_amax(bits.view(np.float32), fmt)
        assert np.array_equal(b, b_ref) and np.array_equal(n.view(np.uint32), n_ref.view(np.uint32))


def test_e8m0_decode_of_every_byte():
    """device/utils.cuh:124-126: scale = (byte << 23) reinterpreted, so byte 0 decodes to 0.0 and byte 255 to +inf."""
    from oracle.codecs import e8m0_decode
    z = _mx()
    assert np.array_equal(e8m0_decode(np.arange(256, dtype=np.uint8)).view(np.uint32), z["e8m0_decode_bits"])


@pytest.mark.parametrize("fmt", ["e4m3", "e5m2"])
def test_mx_dequantize_against_the_reference_torch_dequantizer(fmt):
    z = _mx()
    got = oq.dequantize_mx(z[f"deq_codes_{fmt}"], z[f"deq_scales_{fmt}"], fmt)
    assert np.array_equal(got.view(np.uint32), z[f"deq_out_{fmt}"].view(np.uint32))


def test_mx_padded_layouts():
    """Shapes and pad positions of the row-wise, column-wise and batched MX outputs as the reference's tests fix them
    (dequantized output == zero-padded input within the reference's tolerance, pads exactly zero)."""
    z = _mx()
    for i in range(int(z["n_pad"])):
        fn, axis = str(z[f"pad{i}_fn"]), int(z[f"pad{i}_axis"])
        x, ref = bf16_to_f32(z[f"pad{i}_x_bf16"]), bf16_to_f32(z[f"pad{i}_ref_bf16"])
        fmt, tol = ("e4m3", 1e-1) if fn == "mxfp8_padded_ref" else ("e2m1", 0.5)
        if x.ndim == 2:
            q, s = oq.quantize_mx(x, fmt, axis)
            y = oq.dequantize_mx(q, s, fmt)
            y = y.T if axis == 0 else y          # the column-wise copy is stored transposed; the reference returns [M_pad, N]
        else:
            q, s = oq.quantize_mx_batched(x, fmt, axis)
            y = oq.dequantize_mx(q, s, fmt)      # batched column-wise stays [B, N, M_pad], as in the reference
        assert y.shape == ref.shape, (fn, axis, y.shape, ref.shape)
        assert np.allclose(y, ref, rtol=tol, atol=tol)
        assert np.array_equal(y[ref == 0], ref[ref == 0])
