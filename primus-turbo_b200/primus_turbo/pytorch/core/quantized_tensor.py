"""QuantizedTensor: quantized bytes + scale_inv + the metadata needed to check and undo the quantization.

A light container with the fields and methods the GEMM operators use from the reference's
QuantizedTensor (primus_turbo/pytorch/core/quantized_tensor.py:148-835): qdata, scale_inv,
real_dtype (the quantized dtype), orig_dtype, granularity / axis / block_size / scaling_recipe,
shape (the original, unpadded shape), quantize(), dequantize(), t().
"""
from typing import NamedTuple, Optional

import torch

from .low_precision import (Float4QuantConfig, Float8QuantConfig, ScalingGranularity, ScalingRecipe, is_fp4_dtype)


def _norm_axis(axis, ndim):
    if axis is None:
        return None
    return axis if axis >= 0 else ndim + axis


class QuantizedTensor:
    def __init__(self, qdata, scale_inv, *, orig_dtype, orig_shape, granularity, axis=None, block_size=None,
                 scaling_recipe=None):
        self.qdata = qdata
        self.scale_inv = scale_inv
        self.orig_dtype = orig_dtype
        self._shape = torch.Size(orig_shape)
        self.granularity = granularity
        self.axis = _norm_axis(axis, len(orig_shape))
        self.block_size = block_size
        self.scaling_recipe = scaling_recipe

    # ---- metadata
    @property
    def real_dtype(self):
        return self.qdata.dtype

    @property
    def shape(self):
        return self._shape

    @property
    def dtype(self):
        return self.orig_dtype

    @property
    def device(self):
        return self.qdata.device

    def dim(self):
        return len(self._shape)

    def size(self, i=None):
        return self._shape if i is None else self._shape[i]

    # ---- construction
    @classmethod
    def quantize(cls, x: torch.Tensor, dtype: torch.dtype, granularity: ScalingGranularity, *, axis: Optional[int] = None,
                 block_size: Optional[int] = None, scaling_recipe: Optional[ScalingRecipe] = None) -> "QuantizedTensor":
        from ..ops.quantization import quantize_fp4, quantize_fp8
        if granularity == ScalingGranularity.MX_BLOCKWISE and block_size is None:
            block_size = 32
        fn = quantize_fp4 if is_fp4_dtype(dtype) else quantize_fp8
        q, s = fn(x, dtype, granularity, block_size=block_size, axis=axis, scaling_recipe=scaling_recipe)
        return cls(q, s, orig_dtype=x.dtype, orig_shape=x.shape, granularity=granularity, axis=axis,
                   block_size=block_size, scaling_recipe=scaling_recipe)

    def dequantize(self, dtype: Optional[torch.dtype] = None) -> torch.Tensor:
        from ..ops.quantization import dequantize_fp4, dequantize_fp8
        dtype = dtype or self.orig_dtype
        fn = dequantize_fp4 if is_fp4_dtype(self.qdata.dtype) else dequantize_fp8
        y = fn(self.qdata, dtype, self.granularity, block_size=self.block_size, axis=self.axis,
               scale_inv=self.scale_inv, scaling_recipe=self.scaling_recipe)
        if self.granularity == ScalingGranularity.MX_BLOCKWISE:  # drop the 128-padding
            y = y[..., : self._shape[-2], : self._shape[-1]]
        return y

    def t(self) -> "QuantizedTensor":
        """Transposed view; only tensorwise scaling survives a transpose unchanged
        (quantized_tensor.py:762-764 of the reference)."""
        assert self.granularity == ScalingGranularity.TENSORWISE and self.qdata.dim() == 2, \
            "t() is defined for 2-D tensorwise tensors"
        return QuantizedTensor(self.qdata.t(), self.scale_inv, orig_dtype=self.orig_dtype,
                               orig_shape=self._shape[::-1], granularity=self.granularity)

    def contiguous(self) -> "QuantizedTensor":
        if self.qdata.is_contiguous():
            return self
        from ..kernels.quantization.quantization_impl import transpose_2d
        q = self.qdata
        if q.dim() == 2 and q.t().is_contiguous():
            q = transpose_2d(q.t())  # byte transpose on the device
        else:
            q = q.contiguous()
        return QuantizedTensor(q, self.scale_inv, orig_dtype=self.orig_dtype, orig_shape=self._shape,
                               granularity=self.granularity, axis=self.axis, block_size=self.block_size,
                               scaling_recipe=self.scaling_recipe)

    def __repr__(self):
        return (f"QuantizedTensor(shape={tuple(self._shape)}, real_dtype={self.real_dtype}, orig_dtype={self.orig_dtype}, "
                f"granularity={self.granularity.name}, axis={self.axis}, block_size={self.block_size})")


class QuantizedTensorPair(NamedTuple):
    """A quantized tensor together with the copy quantized along the other axis (used for backward)."""
    data: QuantizedTensor
    data_t: Optional[QuantizedTensor] = None


def check_quantized_tensor(t: QuantizedTensor, config, axis: Optional[int] = None,
                           scaling_recipe: Optional[ScalingRecipe] = None):
    """Strict check that a pre-quantized input matches the GEMM's config
    (core/quantized_tensor.py:113-145 of the reference)."""
    assert isinstance(t, QuantizedTensor)
    assert isinstance(config, (Float8QuantConfig, Float4QuantConfig))
    if t.granularity != config.granularity:
        raise ValueError(f"granularity mismatch: tensor {t.granularity} vs config {config.granularity}")
    if config.granularity in (ScalingGranularity.BLOCKWISE, ScalingGranularity.MX_BLOCKWISE) and t.block_size != config.block_size:
        raise ValueError(f"block_size mismatch: tensor {t.block_size} vs config {config.block_size}")
    if axis is not None and t.axis != _norm_axis(axis, t.dim()):
        raise ValueError(f"axis mismatch: tensor quantized along {t.axis}, GEMM needs {_norm_axis(axis, t.dim())}")
    if scaling_recipe is not None and (t.scaling_recipe or ScalingRecipe()) != scaling_recipe:
        raise ValueError(f"scaling recipe mismatch: tensor {t.scaling_recipe} vs required {scaling_recipe}")
