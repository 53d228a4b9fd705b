"""Formats, granularities and quantization configs of the low-precision GEMM path.

Same names, fields and validation as primus_turbo/pytorch/core/low_precision.py:77-213 of the
reference.  On B200 (compute capability 10.0) the OCP fp8 types are the native ones, so
float8_e4m3 is torch.float8_e4m3fn and float8_e5m2 is torch.float8_e5m2.
"""
from dataclasses import dataclass
from enum import Enum, auto
from typing import NamedTuple, Optional

import torch

float8_e4m3 = torch.float8_e4m3fn
float8_e5m2 = torch.float8_e5m2
float4_e2m1fn_x2 = torch.float4_e2m1fn_x2
float8_e8m0 = torch.float8_e8m0fnu

BLOCKWISE_BLOCK_SIZE = 128
MXFP8_BLOCK_SIZE = 32
MXFP4_BLOCK_SIZE = 32
MX_PADDING_ALIGN_SIZE = 128


def is_fp8_dtype(dtype) -> bool:
    return dtype in (torch.float8_e4m3fn, torch.float8_e5m2)


def is_fp4_dtype(dtype) -> bool:
    return dtype == torch.float4_e2m1fn_x2


class Format(Enum):
    E4M3 = auto()
    E5M2 = auto()
    E2M1_X2 = auto()
    HYBRID = auto()   # e4m3 forward, e5m2 for gradients


class ScaleDtype(Enum):
    FP32 = auto()
    E8M0 = auto()


class ScalingGranularity(Enum):
    TENSORWISE = auto()
    ROWWISE = auto()
    BLOCKWISE = auto()
    MX_BLOCKWISE = auto()


class ScalingStrategy(Enum):
    DYNAMIC = auto()


class ScalingRecipe(NamedTuple):
    """Per-operand options of the MX quantizers (low_precision.py:145-162 of the reference).
    shuffle_scale / shuffle_out: the dense quantizers return the scales / codes in the reference's pre-shuffled tile order
    (what shuffle_scale / shuffle_weight make of the plain outputs).  That order is an export format for the reference's
    pre-shuffled GEMM back ends: the GEMMs of this library read the plain layout only."""
    use_2d_block: bool = False
    use_sr: bool = False
    use_rht: bool = False
    shuffle_scale: bool = False
    shuffle_out: bool = False


@dataclass
class Float8QuantConfig:
    format: Format = Format.E4M3
    granularity: ScalingGranularity = ScalingGranularity.TENSORWISE
    strategy: ScalingStrategy = ScalingStrategy.DYNAMIC
    scale_dtype: ScaleDtype = ScaleDtype.FP32
    block_size: Optional[int] = None

    def __post_init__(self):
        if self.format not in (Format.E4M3, Format.E5M2, Format.HYBRID):
            raise ValueError(f"Float8QuantConfig: unsupported format {self.format}")
        if self.granularity == ScalingGranularity.BLOCKWISE:
            if self.block_size is None:
                raise ValueError("block_size must be set when granularity is BLOCKWISE")
            if self.block_size != BLOCKWISE_BLOCK_SIZE:
                raise ValueError(f"BLOCKWISE supports block_size {BLOCKWISE_BLOCK_SIZE} only")
        if self.granularity == ScalingGranularity.MX_BLOCKWISE:
            if self.block_size is None:
                self.block_size = MXFP8_BLOCK_SIZE
            if self.block_size != MXFP8_BLOCK_SIZE:
                raise ValueError(f"MX_BLOCKWISE requires block_size {MXFP8_BLOCK_SIZE}")
            if self.scale_dtype != ScaleDtype.E8M0:
                raise ValueError("MX_BLOCKWISE requires scale_dtype E8M0")
        elif self.scale_dtype != ScaleDtype.FP32:
            raise ValueError("only MX_BLOCKWISE uses E8M0 scales")


@dataclass
class Float4QuantConfig:
    format: Format = Format.E2M1_X2
    granularity: ScalingGranularity = ScalingGranularity.MX_BLOCKWISE
    strategy: ScalingStrategy = ScalingStrategy.DYNAMIC
    scale_dtype: ScaleDtype = ScaleDtype.E8M0
    block_size: Optional[int] = MXFP4_BLOCK_SIZE
    use_gradient_sr: bool = False   # stochastic rounding when the output gradient is quantized (backward of the FP4 GEMMs)
    use_preshuffle: bool = False    # AITER pre-shuffled layouts: not provided on B200

    def __post_init__(self):
        if self.use_preshuffle:
            raise NotImplementedError("use_preshuffle (AITER pre-shuffled layouts) is not provided by the B200 back end")
        if self.format != Format.E2M1_X2:
            raise ValueError("Float4QuantConfig: format must be E2M1_X2")
        if self.granularity != ScalingGranularity.MX_BLOCKWISE:
            raise ValueError("Float4QuantConfig: granularity must be MX_BLOCKWISE")
        if self.block_size != MXFP4_BLOCK_SIZE:
            raise ValueError(f"Float4QuantConfig: block_size must be {MXFP4_BLOCK_SIZE}")
        if self.scale_dtype != ScaleDtype.E8M0:
            raise ValueError("Float4QuantConfig: scale_dtype must be E8M0")
