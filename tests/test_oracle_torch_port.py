"""The torch-CPU port used as the timed CPU baseline against the numpy oracle, bit for bit."""
import numpy as np
import pytest
import torch

from oracle import quant as oq
from oracle import torch_port as tp


@pytest.mark.parametrize("fmt", ["e4m3", "e5m2"])
@pytest.mark.parametrize("use_2d", [False, True])
def test_mx_rows_match_numpy_oracle(fmt, use_2d):
    g = torch.Generator().manual_seed(7)
    x = torch.randn(256, 384, generator=g)
    x = torch.where(torch.rand(256, 384, generator=g) < 0.01, x * 50, x).to(torch.bfloat16).float()
    x[:32, :64] = 0
    q, s = tp.mx_quantize_rows(x, fmt, use_2d)
    wq, ws = oq.quantize_mx(x.numpy(), fmt, 1, use_2d)
    assert np.array_equal(s.numpy(), ws)
    assert np.array_equal(q.view(torch.uint8).numpy(), wq)
    d = tp.mx_dequantize_rows(q, s).numpy()
    assert np.array_equal(d.view(np.uint32), oq.dequantize_mx(wq, ws, fmt).view(np.uint32))


def test_tensorwise_matches_numpy_oracle():
    x = torch.randn(300, 130, generator=torch.Generator().manual_seed(8)).to(torch.bfloat16)
    q, sinv = tp.tensorwise_quantize(x, "e4m3")
    wq, ws = oq.quantize_fp8_tensorwise(x.float().numpy(), "e4m3")
    assert np.array_equal(q.view(torch.uint8).numpy(), wq)
    assert float(sinv) == float(ws)
