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
