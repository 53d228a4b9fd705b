"""QuantizedTensor: a tensor wrapper subclass that carries quantized bytes + scale_inv + the metadata needed to
check and undo the quantization.

Same role and surface as the reference's QuantizedTensor (primus_turbo/pytorch/core/quantized_tensor.py:148-835):
the wrapper reports the original (unpadded) shape and the original dtype, `qdata` / `scale_inv` hold the
quantized payload, `real_dtype` is the quantized dtype, and the tensor flattens into its inner tensors + metadata
for FSDP / torch.compile.  View-like operations are answered without dequantizing where the scales allow it
(detach / alias / clone always; view / reshape when the scaled trailing dimensions are untouched; t / transpose
for tensorwise scaling, whose single scale survives a transpose).
"""
from typing import NamedTuple, Optional, Tuple, Union

import torch

from .low_precision import (Float4QuantConfig, Float8QuantConfig, ScalingGranularity, ScalingRecipe, is_fp4_dtype)


def _norm_axis(axis, ndim):
    if axis is None:
        return None
    return axis if axis >= 0 else ndim + axis


class QuantizedTensor(torch.Tensor):
    @staticmethod
    def __new__(cls, qdata, scale_inv, *, orig_dtype, orig_shape=None, granularity, axis=None, block_size=None,
                scaling_recipe=None, group_lens=None, group_offs=None, orig_group_lens=None, orig_group_offs=None,
                is_grouped_tensor=None, requires_grad=False, shape=None, dest_dtype=None, quantized_axis=None):
        # `shape`, `dest_dtype`, `quantized_axis` are the reference's keyword names for orig_shape, the quantized
        # dtype (always qdata.dtype here) and axis.  A grouped tensor (MoE activations, groups along dim 0) carries
        # the tight group_lens / offs of the source (orig_*) and those of its padded payload (group_*).
        orig_shape = torch.Size(orig_shape if orig_shape is not None else shape)
        if axis is None:
            axis = quantized_axis
        assert dest_dtype is None or dest_dtype == qdata.dtype, "dest_dtype must be the dtype of the quantized data"
        self = torch.Tensor._make_wrapper_subclass(cls, orig_shape, dtype=orig_dtype, layout=qdata.layout,
                                                   device=qdata.device, requires_grad=requires_grad)
        self._qdata, self._scale_inv = qdata, scale_inv
        self._granularity = granularity
        self._axis = _norm_axis(axis, len(orig_shape))
        self._block_size = block_size
        self._scaling_recipe = scaling_recipe
        self._group_lens, self._group_offs = group_lens, group_offs
        self._orig_group_lens, self._orig_group_offs = orig_group_lens, orig_group_offs
        self._is_grouped_tensor = bool(is_grouped_tensor) if is_grouped_tensor is not None else group_lens is not None
        return self

    def __init__(self, *args, **kwargs):
        pass

    # ---- payload and metadata
    @property
    def qdata(self):
        return self._qdata

    @property
    def scale_inv(self):
        return self._scale_inv

    @property
    def real_dtype(self):
        return self._qdata.dtype

    @property
    def orig_dtype(self):
        return self.dtype

    @property
    def granularity(self):
        return self._granularity

    @property
    def axis(self):
        return self._axis

    quantized_axis = axis

    @property
    def block_size(self):
        return self._block_size

    @property
    def scaling_recipe(self):
        return self._scaling_recipe

    @property
    def group_lens(self):
        return self._group_lens

    @property
    def group_offs(self):
        return self._group_offs

    @property
    def orig_group_lens(self):
        return self._orig_group_lens

    @property
    def orig_group_offs(self):
        return self._orig_group_offs

    @property
    def is_grouped_tensor(self):
        return self._is_grouped_tensor

    def _like(self, qdata, scale_inv, shape, axis="same"):
        return QuantizedTensor(qdata, scale_inv, orig_dtype=self.dtype, orig_shape=shape, granularity=self._granularity,
                               axis=self._axis if axis == "same" else axis, block_size=self._block_size,
                               scaling_recipe=self._scaling_recipe, group_lens=self._group_lens,
                               group_offs=self._group_offs, orig_group_lens=self._orig_group_lens,
                               orig_group_offs=self._orig_group_offs, is_grouped_tensor=self._is_grouped_tensor,
                               requires_grad=False)

    # ---- construction
    @classmethod
    def quantize(cls, x: torch.Tensor, dtype: torch.dtype, granularity: ScalingGranularity, *, axis: Optional[int] = None,
                 block_size: Optional[int] = None, scaling_recipe: Optional[ScalingRecipe] = None,
                 group_lens: Optional[torch.Tensor] = None) -> "QuantizedTensor":
        """With `group_lens` (int64 on the device) x is a grouped tensor [total_m, N].  Tensorwise / rowwise treat it
        as one tensor and only record the groups; MX quantizes group by group into the padded layout the grouped
        GEMMs read (primus_turbo/pytorch/core/quantized_tensor.py:300-343 of the reference)."""
        from ..ops.quantization import grouped_quantize_fp4, grouped_quantize_fp8, quantize_fp4, quantize_fp8
        if granularity == ScalingGranularity.MX_BLOCKWISE and block_size is None:
            block_size = 32
        fp4 = is_fp4_dtype(dtype)
        grouped = group_lens is not None
        meta = {}
        with torch.no_grad():
            if grouped:
                from ..kernels.grouped_gemm.grouped_gemm_utils import group_offs_from_lens
                assert group_lens.is_cuda, "group_lens must be on CUDA"
                offs = group_offs_from_lens(group_lens)
                meta = dict(orig_group_lens=group_lens, orig_group_offs=offs, is_grouped_tensor=True)
            if grouped and granularity not in (ScalingGranularity.TENSORWISE, ScalingGranularity.ROWWISE):
                fn = grouped_quantize_fp4 if fp4 else grouped_quantize_fp8
                q, s, plens, poffs = fn(x, dtype, granularity, group_lens, offs, block_size=block_size, axis=axis,
                                        scaling_recipe=scaling_recipe)
                meta.update(group_lens=plens, group_offs=poffs)
            else:
                fn = quantize_fp4 if fp4 else quantize_fp8
                q, s = fn(x, dtype, granularity, block_size=block_size, axis=axis, scaling_recipe=scaling_recipe)
                if grouped:
                    meta.update(group_lens=group_lens, group_offs=offs)
        return cls(q, s, orig_dtype=x.dtype, orig_shape=x.shape, granularity=granularity, axis=axis,
                   block_size=block_size, scaling_recipe=scaling_recipe, **meta)

    def dequantize(self, dtype: Optional[torch.dtype] = None) -> torch.Tensor:
        from ..ops.quantization import dequantize_fp4, dequantize_fp8, grouped_dequantize_fp4, grouped_dequantize_fp8
        dtype = dtype or self.dtype
        fp4 = is_fp4_dtype(self._qdata.dtype)
        mx = self._granularity == ScalingGranularity.MX_BLOCKWISE
        with torch.no_grad():
            if self._is_grouped_tensor and mx and not fp4:
                y = grouped_dequantize_fp8(self._qdata, dtype, self._granularity, self._orig_group_offs, self._group_offs,
                                           block_size=self._block_size, axis=self._axis, scale_inv=self._scale_inv,
                                           scaling_recipe=self._scaling_recipe, total_M=self.shape[0])
            elif self._is_grouped_tensor and mx:
                assert self._axis == self.dim() - 1, "grouped FP4 dequantization is row-wise only"
                y = grouped_dequantize_fp4(self._qdata, dtype, self._granularity, block_size=self._block_size,
                                           axis=self._axis, scale_inv=self._scale_inv, scaling_recipe=self._scaling_recipe)
            else:
                fn = dequantize_fp4 if fp4 else dequantize_fp8
                y = fn(self._qdata, dtype, self._granularity, block_size=self._block_size, axis=self._axis,
                       scale_inv=self._scale_inv, scaling_recipe=self._scaling_recipe)
        if mx:  # drop the 128-padding
            y = y[..., : self.shape[-2], : self.shape[-1]]
        return y

    def contiguous(self) -> "QuantizedTensor":
        """Materialises a lazily transposed payload (byte transpose on the device)."""
        q = self._qdata
        if q.is_contiguous():
            return self
        from ..kernels.quantization.quantization_impl import transpose_2d
        q = transpose_2d(q.t()) if (q.dim() == 2 and q.t().is_contiguous()) else q.contiguous()
        return self._like(q, self._scale_inv, self.shape)

    # ---- flatten / unflatten (FSDP, torch.compile)
    def __tensor_flatten__(self):
        inner = ["_qdata", "_scale_inv"]
        if self._group_lens is not None:
            inner.append("_group_lens")
        if self._group_offs is not None:
            inner.append("_group_offs")
        if self._orig_group_lens is not None:
            inner.append("_orig_group_lens")
        if self._orig_group_offs is not None:
            inner.append("_orig_group_offs")
        meta = dict(granularity=self._granularity, axis=self._axis, block_size=self._block_size,
                    scaling_recipe=self._scaling_recipe, orig_dtype=self.dtype, is_grouped_tensor=self._is_grouped_tensor)
        return inner, meta

    @staticmethod
    def __tensor_unflatten__(inner_tensors, meta, outer_size, outer_stride):
        return QuantizedTensor(inner_tensors["_qdata"], inner_tensors["_scale_inv"], orig_dtype=meta["orig_dtype"],
                               orig_shape=outer_size, granularity=meta["granularity"], axis=meta["axis"],
                               block_size=meta["block_size"], scaling_recipe=meta["scaling_recipe"],
                               group_lens=inner_tensors.get("_group_lens"), group_offs=inner_tensors.get("_group_offs"),
                               orig_group_lens=inner_tensors.get("_orig_group_lens"),
                               orig_group_offs=inner_tensors.get("_orig_group_offs"),
                               is_grouped_tensor=meta.get("is_grouped_tensor"))

    # ---- view-like operations that keep the quantization valid
    def _reshaped(self, shape, op):
        """view / reshape to `shape` when the scales stay attached to the same elements: tensorwise always; otherwise
        the trailing dimensions the scales refer to (the last one for rowwise along the last axis, the last two for
        every other case) must be unchanged, and the leading ones are regrouped alike on data and scales."""
        shape = list(shape[0]) if len(shape) == 1 and isinstance(shape[0], (tuple, list, torch.Size)) else list(shape)
        numel = self.numel()
        if -1 in shape:
            known = 1
            for d in shape:
                known *= d if d != -1 else 1
            shape[shape.index(-1)] = numel // max(known, 1)
        new_shape = torch.Size(shape)
        q, s = self._qdata, self._scale_inv
        if self._granularity == ScalingGranularity.TENSORWISE:
            return self._like(op(q, new_shape), s, new_shape)
        keep = 1 if (self._granularity == ScalingGranularity.ROWWISE and self._axis == self.dim() - 1) else 2
        if len(new_shape) < keep or tuple(new_shape[-keep:]) != tuple(self.shape[-keep:]):
            raise NotImplementedError(f"QuantizedTensor: cannot view {tuple(self.shape)} as {tuple(new_shape)} without "
                                      f"dequantizing ({self._granularity.name} scales are tied to the trailing dimensions)")
        lead = tuple(new_shape[:-keep])
        axis = None if self._axis is None else len(new_shape) - (self.dim() - self._axis)
        return self._like(op(q, lead + tuple(q.shape[-keep:])), op(s, lead + tuple(s.shape[-keep:])), new_shape, axis=axis)

    @classmethod
    def __torch_dispatch__(cls, func, types, args=(), kwargs=None):
        aten = torch.ops.aten
        t = args[0]
        if func in (aten.detach.default, aten.alias.default):
            return t._like(t._qdata.detach(), t._scale_inv.detach(), t.shape)
        if func is aten.clone.default:
            return t._like(t._qdata.clone(), t._scale_inv.clone(), t.shape)
        if func in (aten.view.default, aten._unsafe_view.default):
            return t._reshaped((args[1],), torch.Tensor.view)
        if func is aten.reshape.default:
            return t._reshaped((args[1],), torch.Tensor.reshape)
        if func in (aten.t.default, aten.transpose.int):
            d0, d1 = (0, 1) if func is aten.t.default else (args[1] % t.dim(), args[2] % t.dim())
            if t._granularity != ScalingGranularity.TENSORWISE or t.dim() != 2:
                raise NotImplementedError("QuantizedTensor: only 2-D tensorwise tensors transpose without requantizing "
                                          "(quantized_tensor.py:762-764 of the reference)")
            if d0 == d1:
                return t
            return t._like(t._qdata.t(), t._scale_inv, t.shape[::-1])   # lazy: .contiguous() moves the bytes
        raise NotImplementedError(f"QuantizedTensor: {func} needs the values; call dequantize() first")

    __torch_function__ = torch._C._disabled_torch_function_impl

    def __repr__(self, *, tensor_contents=None):
        return (f"QuantizedTensor(shape={tuple(self.shape)}, real_dtype={self.real_dtype}, orig_dtype={self.dtype}, "
                f"granularity={self._granularity.name}, axis={self._axis}, block_size={self._block_size})")


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


def create_quantized_weight(weight: torch.Tensor, dest_dtype: torch.dtype,
                            quant_config: Union[Float4QuantConfig, Float8QuantConfig],
                            need_weight_transpose_cache: bool = False) -> Tuple[QuantizedTensor, Optional[QuantizedTensor]]:
    """Quantizes a weight ([N, K] or [G, N, K]) once so that GEMM calls can reuse it: returns (weight_q, weight_q_t) where
    weight_q is what the forward GEMM reads and weight_q_t the copy backward needs (None unless asked for).  Same call as
    create_quantized_weight of the reference (primus_turbo/pytorch/core/quantized_tensor.py:897-956): 2-D block scales
    for BLOCKWISE / MX weights and FP4, plain scales otherwise.  weight_q_t per recipe: TENSORWISE the lazily transposed
    view (2-D weights; the single scale survives a transpose); ROWWISE the weight scaled along its other axis in the
    same layout, which is the operand FP8GemmRowFunction / FP8GroupedGemmRowFunc take as `b_t`; BLOCKWISE / MX the
    quantization along axis -2."""
    if isinstance(quant_config, Float4QuantConfig):
        if getattr(quant_config, "use_preshuffle", False):
            raise NotImplementedError("pre-shuffled weight layouts are not provided on B200")
        recipe = ScalingRecipe(use_2d_block=True)
    elif quant_config.granularity in (ScalingGranularity.BLOCKWISE, ScalingGranularity.MX_BLOCKWISE):
        recipe = ScalingRecipe(use_2d_block=True)
    else:
        recipe = ScalingRecipe()
    gran, bs = quant_config.granularity, quant_config.block_size
    weight = weight.detach()
    qw = QuantizedTensor.quantize(weight, dest_dtype, gran, axis=-1, block_size=bs, scaling_recipe=recipe)
    qw_t = None
    if need_weight_transpose_cache:
        if gran == ScalingGranularity.TENSORWISE:
            qw_t = qw.transpose(-2, -1) if weight.dim() == 2 else None
        elif gran in (ScalingGranularity.ROWWISE, ScalingGranularity.BLOCKWISE, ScalingGranularity.MX_BLOCKWISE):
            qw_t = QuantizedTensor.quantize(weight, dest_dtype, gran, axis=-2, block_size=bs, scaling_recipe=recipe)
        else:
            raise ValueError(f"Unsupported granularity: {gran}")
    return qw, qw_t
