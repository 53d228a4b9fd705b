"""QuantizedTensor as a tensor wrapper subclass: metadata, view rules, flatten / unflatten, config checks.
Mirrors what tests/pytorch/core/test_quantized_tensor.py:116-609 of the reference asserts about shape and metadata
handling; no kernel runs here (payloads are built by hand on the CPU)."""
import pytest
import torch

from primus_turbo.pytorch.core.low_precision import (Float8QuantConfig, Format, ScaleDtype, ScalingGranularity as SG,
                                                     ScalingRecipe)
from primus_turbo.pytorch.core.quantized_tensor import QuantizedTensor, QuantizedTensorPair, check_quantized_tensor

F8 = torch.float8_e4m3fn


def _payload(*shape):
    return torch.arange(int(torch.Size(shape).numel()), dtype=torch.int64).remainder(120).to(torch.uint8).view(*shape).view(F8)


def test_wrapper_reports_original_shape_and_dtype():
    # MX data is padded to 128 columns, the wrapper keeps the unpadded shape (quantized_tensor.py:353-355 of the reference)
    q, s = _payload(200, 128), torch.full((200, 4), 127, dtype=torch.uint8)
    t = QuantizedTensor(q, s, orig_dtype=torch.bfloat16, orig_shape=(200, 96), granularity=SG.MX_BLOCKWISE, axis=-1, block_size=32)
    assert isinstance(t, torch.Tensor) and t.shape == (200, 96) and t.dtype == torch.bfloat16
    assert t.real_dtype == F8 and t.qdata is q and t.scale_inv is s and t.axis == 1 and t.quantized_axis == 1
    assert t.granularity == SG.MX_BLOCKWISE and t.block_size == 32 and not t.requires_grad
    assert "MX_BLOCKWISE" in repr(t)


def test_reference_keyword_names_are_accepted():
    q, s = _payload(8, 16), torch.ones(8, 1)
    t = QuantizedTensor(q, s, shape=torch.Size((8, 16)), orig_dtype=torch.float16, dest_dtype=F8, granularity=SG.ROWWISE,
                        quantized_axis=-1)
    assert t.shape == (8, 16) and t.axis == 1
    with pytest.raises(AssertionError):
        QuantizedTensor(q, s, shape=(8, 16), orig_dtype=torch.float16, dest_dtype=torch.float8_e5m2, granularity=SG.ROWWISE)


def test_detach_alias_clone_keep_metadata():
    q, s = _payload(4, 8), torch.ones(())
    t = QuantizedTensor(q, s, orig_dtype=torch.bfloat16, orig_shape=(4, 8), granularity=SG.TENSORWISE)
    d, c = t.detach(), t.clone()
    for u in (d, c):
        assert isinstance(u, QuantizedTensor) and u.shape == t.shape and u.granularity == SG.TENSORWISE
    assert d.qdata.data_ptr() == q.data_ptr() and c.qdata.data_ptr() != q.data_ptr()
    assert torch.equal(c.qdata.view(torch.uint8), q.view(torch.uint8))


def test_view_rules_follow_the_scales():
    # tensorwise: one scale, any view
    t = QuantizedTensor(_payload(4, 6, 8), torch.ones(()), orig_dtype=torch.bfloat16, orig_shape=(4, 6, 8), granularity=SG.TENSORWISE)
    assert t.view(24, 8).shape == (24, 8) and t.reshape(4, 48).qdata.shape == (4, 48) and t.view(-1, 8).shape == (24, 8)
    # rowwise along the last axis: leading dimensions regroup, data and scales alike
    r = QuantizedTensor(_payload(4, 6, 8), torch.ones(4, 6, 1), orig_dtype=torch.bfloat16, orig_shape=(4, 6, 8), granularity=SG.ROWWISE, axis=-1)
    v = r.view(24, 8)
    assert v.qdata.shape == (24, 8) and v.scale_inv.shape == (24, 1) and v.axis == 1
    with pytest.raises(NotImplementedError):
        r.view(4, 48)
    # blockwise: the last two dimensions carry the block structure
    b = QuantizedTensor(_payload(2, 3, 128, 256), torch.ones(2, 3, 128, 2), orig_dtype=torch.bfloat16, orig_shape=(2, 3, 128, 256),
                        granularity=SG.BLOCKWISE, axis=-1, block_size=128)
    vb = b.view(6, 128, 256)
    assert vb.scale_inv.shape == (6, 128, 2) and vb.axis == 2
    with pytest.raises(NotImplementedError):
        b.view(2, 3, 256, 128)


def test_transpose_only_for_tensorwise():
    t = QuantizedTensor(_payload(4, 8), torch.ones(()), orig_dtype=torch.bfloat16, orig_shape=(4, 8), granularity=SG.TENSORWISE)
    tt = t.t()
    assert tt.shape == (8, 4) and not tt.qdata.is_contiguous() and tt.scale_inv is not None
    assert torch.equal(tt.qdata.view(torch.uint8), t.qdata.view(torch.uint8).t())
    r = QuantizedTensor(_payload(4, 8), torch.ones(4, 1), orig_dtype=torch.bfloat16, orig_shape=(4, 8), granularity=SG.ROWWISE, axis=-1)
    with pytest.raises(NotImplementedError):
        r.t()


def test_value_operations_are_refused():
    t = QuantizedTensor(_payload(4, 8), torch.ones(()), orig_dtype=torch.bfloat16, orig_shape=(4, 8), granularity=SG.TENSORWISE)
    with pytest.raises(NotImplementedError):
        t + 1


def test_flatten_unflatten_round_trip():
    lens = torch.tensor([3, 5]); offs = torch.tensor([0, 3, 8])
    t = QuantizedTensor(_payload(8, 128), torch.full((8, 4), 127, dtype=torch.uint8), orig_dtype=torch.bfloat16, orig_shape=(8, 100),
                        granularity=SG.MX_BLOCKWISE, axis=-1, block_size=32, scaling_recipe=ScalingRecipe(use_2d_block=True),
                        group_lens=lens, group_offs=offs)
    names, meta = t.__tensor_flatten__()
    assert names == ["_qdata", "_scale_inv", "_group_lens", "_group_offs"]
    u = QuantizedTensor.__tensor_unflatten__({n: getattr(t, n) for n in names}, meta, t.shape, t.stride())
    assert u.shape == t.shape and u.dtype == t.dtype and u.granularity == t.granularity and u.axis == t.axis
    assert u.block_size == 32 and u.scaling_recipe == t.scaling_recipe and u.qdata is t.qdata and u.group_offs is offs


def test_check_quantized_tensor_is_strict():
    cfg = Float8QuantConfig(format=Format.E4M3, granularity=SG.MX_BLOCKWISE, scale_dtype=ScaleDtype.E8M0, block_size=32)
    t = QuantizedTensor(_payload(8, 128), torch.full((8, 4), 127, dtype=torch.uint8), orig_dtype=torch.bfloat16, orig_shape=(8, 128),
                        granularity=SG.MX_BLOCKWISE, axis=-1, block_size=32)
    check_quantized_tensor(t, cfg, axis=-1)
    with pytest.raises(ValueError):
        check_quantized_tensor(t, cfg, axis=0)
    with pytest.raises(ValueError):
        check_quantized_tensor(t, Float8QuantConfig(granularity=SG.TENSORWISE))
    with pytest.raises(ValueError):
        check_quantized_tensor(t, cfg, scaling_recipe=ScalingRecipe(use_2d_block=True))
    pair = QuantizedTensorPair(t)
    assert pair.data is t and pair.data_t is None
