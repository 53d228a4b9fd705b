"""torch.library registrations: `torch.ops.primus_turbo.*` with fake (meta) implementations.

The reference exposes its GEMM and blockwise-quantize entry points as custom ops so that they can be traced, exported and
compiled (primus_turbo/pytorch/kernels/gemm/gemm_fp8_impl.py:518-633, gemm_fp4_impl.py:339-441, gemm_impl.py:120-200,
kernels/grouped_gemm/grouped_gemm_fp8_impl.py:888-1110, grouped_gemm_fp4_impl.py:429-560, grouped_gemm_impl.py:476-620,
kernels/quantization/quantization_impl.py:81-490).  The same names and schemas are registered here: `granularity` and
`default_backend` travel as ints (`default_backend` is accepted and ignored, there is one back end), every op is CUDA-only,
and each has a `register_fake` that gives the output shapes without touching a device.  The real implementations are the
functions of the `*_impl` modules, which call the C ABI.

The autograd Functions of `primus_turbo.pytorch.ops` call those functions directly (one Python frame less per launch);
code that was written against `torch.ops.primus_turbo.<name>` or traces through the ops finds them here.
"""
from typing import List, Optional, Tuple

import torch

from .gemm import gemm_fp4_impl as _g4
from .gemm import gemm_fp8_impl as _g8
from .gemm import gemm_impl as _g16
from .grouped_gemm import grouped_gemm_fp4_impl as _gg4
from .grouped_gemm import grouped_gemm_fp8_impl as _gg8
from .grouped_gemm import grouped_gemm_impl as _gg16
from .quantization import quantization_impl as _q

_op = torch.library.custom_op
BLOCK = 128


def _ceil_div(a, b):
    return (a + b - 1) // b


def _logical_mn(a, b, trans_a, trans_b):
    return (a.shape[1] if trans_a else a.shape[0]), (b.shape[0] if trans_b else b.shape[1])


def _out2d(a, b, trans_a, trans_b, trans_c, out_dtype):
    m, n = _logical_mn(a, b, trans_a, trans_b)
    return torch.empty((n, m) if trans_c else (m, n), dtype=out_dtype, device=a.device)


# ------------------------------------------------------------------------------------------------ dense GEMMs
@_op("primus_turbo::gemm_fp8_impl", mutates_args=(), device_types="cuda")
def gemm_fp8_impl(a: torch.Tensor, a_scale_inv: torch.Tensor, trans_a: bool, b: torch.Tensor, b_scale_inv: torch.Tensor,
                  trans_b: bool, out_dtype: torch.dtype, trans_c: bool, granularity: int, default_backend: int) -> torch.Tensor:
    return _g8.gemm_fp8_impl(a, a_scale_inv, trans_a, b, b_scale_inv, trans_b, out_dtype, trans_c, granularity)


@gemm_fp8_impl.register_fake
def _(a, a_scale_inv, trans_a, b, b_scale_inv, trans_b, out_dtype, trans_c, granularity, default_backend):
    return _out2d(a, b, trans_a, trans_b, trans_c, out_dtype)


@_op("primus_turbo::gemm_fp8_accum_impl", mutates_args={"out"}, device_types="cuda")
def gemm_fp8_accum_impl(a: torch.Tensor, a_scale_inv: torch.Tensor, trans_a: bool, b: torch.Tensor, b_scale_inv: torch.Tensor,
                        trans_b: bool, out_dtype: torch.dtype, trans_c: bool, granularity: int, out: torch.Tensor,
                        default_backend: int) -> None:
    _g8.gemm_fp8_accum_impl(a, a_scale_inv, trans_a, b, b_scale_inv, trans_b, out, trans_c, granularity)


@gemm_fp8_accum_impl.register_fake
def _(a, a_scale_inv, trans_a, b, b_scale_inv, trans_b, out_dtype, trans_c, granularity, out, default_backend):
    m, n = _logical_mn(a, b, trans_a, trans_b)
    assert tuple(out.shape) == ((n, m) if trans_c else (m, n)), f"out shape {tuple(out.shape)} does not match the product"
    return None


@_op("primus_turbo::gemm_fp4_impl", mutates_args=(), device_types="cuda")
def gemm_fp4_impl(a: torch.Tensor, a_scale_inv: torch.Tensor, trans_a: bool, b: torch.Tensor, b_scale_inv: torch.Tensor,
                  trans_b: bool, out_dtype: torch.dtype, trans_c: bool, granularity: int, default_backend: int,
                  preshuffled: bool = False) -> torch.Tensor:
    return _g4.gemm_fp4_impl(a, a_scale_inv, trans_a, b, b_scale_inv, trans_b, out_dtype, trans_c, granularity, default_backend,
                             preshuffled)


@gemm_fp4_impl.register_fake
def _(a, a_scale_inv, trans_a, b, b_scale_inv, trans_b, out_dtype, trans_c, granularity, default_backend, preshuffled=False):
    m, n = a.shape[0], b.shape[0]     # NT only: both operands are [rows, K / 2] packed
    return torch.empty((n, m) if trans_c else (m, n), dtype=out_dtype, device=a.device)


@_op("primus_turbo::gemm_fp4_accum_impl", mutates_args={"out"}, device_types="cuda")
def gemm_fp4_accum_impl(a: torch.Tensor, a_scale_inv: torch.Tensor, trans_a: bool, b: torch.Tensor, b_scale_inv: torch.Tensor,
                        trans_b: bool, out_dtype: torch.dtype, trans_c: bool, granularity: int, out: torch.Tensor,
                        default_backend: int, preshuffled: bool = False) -> None:
    _g4.gemm_fp4_accum_impl(a, a_scale_inv, trans_a, b, b_scale_inv, trans_b, out, trans_c, granularity, default_backend, preshuffled)


@gemm_fp4_accum_impl.register_fake
def _(a, a_scale_inv, trans_a, b, b_scale_inv, trans_b, out_dtype, trans_c, granularity, out, default_backend, preshuffled=False):
    return None


@_op("primus_turbo::gemm_impl", mutates_args=(), device_types="cuda")
def gemm_impl(a: torch.Tensor, trans_a: bool, b: torch.Tensor, trans_b: bool, out_dtype: torch.dtype, trans_c: bool,
              default_backend: int) -> torch.Tensor:
    return _g16.gemm_impl(a, trans_a, b, trans_b, out_dtype, trans_c)


@gemm_impl.register_fake
def _(a, trans_a, b, trans_b, out_dtype, trans_c, default_backend):
    return _out2d(a, b, trans_a, trans_b, trans_c, out_dtype)


@_op("primus_turbo::gemm_accum_impl", mutates_args={"out"}, device_types="cuda")
def gemm_accum_impl(a: torch.Tensor, trans_a: bool, b: torch.Tensor, trans_b: bool, out_dtype: torch.dtype, trans_c: bool,
                    out: torch.Tensor, default_backend: int) -> None:
    _g16.gemm_accum_impl(a, trans_a, b, trans_b, out_dtype, trans_c, out)


@gemm_accum_impl.register_fake
def _(a, trans_a, b, trans_b, out_dtype, trans_c, out, default_backend):
    return None


# ------------------------------------------------------------------------------------------------ grouped GEMMs
def _grouped_out(a, b, trans_b, out_dtype):
    n = b.shape[1] if trans_b else b.shape[2]
    return torch.empty((a.shape[0], n), dtype=out_dtype, device=a.device)


def _variable_k_out(a, b, trans_a, trans_c, group_lens, out_dtype, blockwise_or_hp):
    """[G, rows_a, rows_b] of the per-group products (operands token-major [T, R] when `blockwise_or_hp`, else [R, T])."""
    ra = a.shape[1] if blockwise_or_hp else a.shape[0]
    rb = b.shape[1] if blockwise_or_hp else b.shape[0]
    g = group_lens.shape[0]
    return torch.empty((g, rb, ra) if trans_c else (g, ra, rb), dtype=out_dtype, device=a.device)


@_op("primus_turbo::grouped_gemm_fp8_impl", mutates_args=(), device_types="cuda")
def grouped_gemm_fp8_impl(a: torch.Tensor, b: torch.Tensor, a_scales: torch.Tensor, b_scales: torch.Tensor, group_lens: torch.Tensor,
                          group_offs: torch.Tensor, trans_a: bool, trans_b: bool, out_dtype: torch.dtype, granularity: int,
                          num_cu: Optional[int], default_backend: int, maybe_pre_sync: bool = False,
                          group_offs_out: Optional[torch.Tensor] = None) -> torch.Tensor:
    return _gg8.grouped_gemm_fp8_impl(a, b, a_scales, b_scales, group_lens, group_offs, trans_a, trans_b, out_dtype, granularity, num_cu,
                                      default_backend, maybe_pre_sync, group_offs_out)


@grouped_gemm_fp8_impl.register_fake
def _(a, b, a_scales, b_scales, group_lens, group_offs, trans_a, trans_b, out_dtype, granularity, num_cu, default_backend,
      maybe_pre_sync=False, group_offs_out=None):
    return _grouped_out(a, b, trans_b, out_dtype)


@_op("primus_turbo::grouped_gemm_fp8_variable_k_impl", mutates_args=(), device_types="cuda")
def grouped_gemm_fp8_variable_k_impl(a: torch.Tensor, b: torch.Tensor, a_scales: torch.Tensor, b_scales: torch.Tensor,
                                     group_lens: torch.Tensor, group_offs: torch.Tensor, trans_a: bool, trans_b: bool, trans_c: bool,
                                     out_dtype: torch.dtype, granularity: int, num_cu: Optional[int], default_backend: int,
                                     maybe_pre_sync: bool = False) -> torch.Tensor:
    return _gg8.grouped_gemm_fp8_variable_k_impl(a, b, a_scales, b_scales, group_lens, group_offs, trans_a, trans_b, trans_c, out_dtype,
                                                 granularity, num_cu, default_backend)


@grouped_gemm_fp8_variable_k_impl.register_fake
def _(a, b, a_scales, b_scales, group_lens, group_offs, trans_a, trans_b, trans_c, out_dtype, granularity, num_cu, default_backend,
      maybe_pre_sync=False):
    return _variable_k_out(a, b, trans_a, trans_c, group_lens, out_dtype, trans_a)


@_op("primus_turbo::grouped_gemm_fp8_variable_k_accum_impl", mutates_args={"out"}, device_types="cuda")
def grouped_gemm_fp8_variable_k_accum_impl(a: torch.Tensor, b: torch.Tensor, a_scales: torch.Tensor, b_scales: torch.Tensor,
                                           group_lens: torch.Tensor, group_offs: torch.Tensor, trans_a: bool, trans_b: bool,
                                           trans_c: bool, out_dtype: torch.dtype, granularity: int, num_cu: Optional[int],
                                           default_backend: int, out: torch.Tensor, maybe_pre_sync: bool = False) -> None:
    _gg8.grouped_gemm_fp8_variable_k_accum_impl(a, b, a_scales, b_scales, group_lens, group_offs, trans_a, trans_b, trans_c, out,
                                                granularity, num_cu, default_backend)


@grouped_gemm_fp8_variable_k_accum_impl.register_fake
def _(a, b, a_scales, b_scales, group_lens, group_offs, trans_a, trans_b, trans_c, out_dtype, granularity, num_cu, default_backend, out,
      maybe_pre_sync=False):
    return None


@_op("primus_turbo::grouped_gemm_fp4_impl", mutates_args=(), device_types="cuda")
def grouped_gemm_fp4_impl(a: torch.Tensor, b: torch.Tensor, a_scales: torch.Tensor, b_scales: torch.Tensor, group_lens: torch.Tensor,
                          group_offs: torch.Tensor, trans_a: bool, trans_b: bool, out_dtype: torch.dtype, granularity: int,
                          num_cu: Optional[int], default_backend: int, maybe_pre_sync: bool = False,
                          group_offs_out: Optional[torch.Tensor] = None) -> torch.Tensor:
    return _gg4.grouped_gemm_fp4_impl(a, b, a_scales, b_scales, group_lens, group_offs, trans_a, trans_b, out_dtype, granularity, num_cu,
                                      default_backend, group_offs_out)


@grouped_gemm_fp4_impl.register_fake
def _(a, b, a_scales, b_scales, group_lens, group_offs, trans_a, trans_b, out_dtype, granularity, num_cu, default_backend,
      maybe_pre_sync=False, group_offs_out=None):
    return torch.empty((a.shape[0], b.shape[1]), dtype=out_dtype, device=a.device)


@_op("primus_turbo::grouped_gemm_fp4_variable_k_impl", mutates_args=(), device_types="cuda")
def grouped_gemm_fp4_variable_k_impl(a: torch.Tensor, b: torch.Tensor, a_scales: torch.Tensor, b_scales: torch.Tensor,
                                     group_lens: torch.Tensor, group_offs: torch.Tensor, trans_a: bool, trans_b: bool, trans_c: bool,
                                     out_dtype: torch.dtype, granularity: int, num_cu: Optional[int], default_backend: int,
                                     maybe_pre_sync: bool = False) -> torch.Tensor:
    lhs, lhs_s, rhs, rhs_s = (b, b_scales, a, a_scales) if trans_c else (a, a_scales, b, b_scales)
    return _gg4.grouped_gemm_fp4_variable_k_impl(lhs, rhs, lhs_s, rhs_s, group_lens, group_offs, out_dtype, granularity, num_cu,
                                                 default_backend)


@grouped_gemm_fp4_variable_k_impl.register_fake
def _(a, b, a_scales, b_scales, group_lens, group_offs, trans_a, trans_b, trans_c, out_dtype, granularity, num_cu, default_backend,
      maybe_pre_sync=False):
    return _variable_k_out(a, b, trans_a, trans_c, group_lens, out_dtype, False)


@_op("primus_turbo::grouped_gemm_fp4_variable_k_accum_impl", mutates_args={"out"}, device_types="cuda")
def grouped_gemm_fp4_variable_k_accum_impl(a: torch.Tensor, b: torch.Tensor, a_scales: torch.Tensor, b_scales: torch.Tensor,
                                           group_lens: torch.Tensor, group_offs: torch.Tensor, trans_a: bool, trans_b: bool,
                                           trans_c: bool, out_dtype: torch.dtype, granularity: int, num_cu: Optional[int],
                                           default_backend: int, out: torch.Tensor, maybe_pre_sync: bool = False) -> None:
    lhs, lhs_s, rhs, rhs_s = (b, b_scales, a, a_scales) if trans_c else (a, a_scales, b, b_scales)
    _gg4.grouped_gemm_fp4_variable_k_accum_impl(lhs, rhs, lhs_s, rhs_s, group_lens, group_offs, out, granularity, num_cu, default_backend)


@grouped_gemm_fp4_variable_k_accum_impl.register_fake
def _(a, b, a_scales, b_scales, group_lens, group_offs, trans_a, trans_b, trans_c, out_dtype, granularity, num_cu, default_backend, out,
      maybe_pre_sync=False):
    return None


@_op("primus_turbo::grouped_gemm_impl", mutates_args=(), device_types="cuda")
def grouped_gemm_impl(a: torch.Tensor, b: torch.Tensor, group_lens: torch.Tensor, group_offs: torch.Tensor, trans_a: bool, trans_b: bool,
                      num_cu: Optional[int], default_backend: int, maybe_pre_sync: bool = False, schedule: str = "static") -> torch.Tensor:
    return _gg16.grouped_gemm_impl(a, b, group_lens, group_offs, trans_a, trans_b, num_cu, default_backend, maybe_pre_sync, schedule)


@grouped_gemm_impl.register_fake
def _(a, b, group_lens, group_offs, trans_a, trans_b, num_cu, default_backend, maybe_pre_sync=False, schedule="static"):
    return _grouped_out(a, b, trans_b, a.dtype)


@_op("primus_turbo::grouped_gemm_variable_k_impl", mutates_args=(), device_types="cuda")
def grouped_gemm_variable_k_impl(a: torch.Tensor, b: torch.Tensor, group_lens: torch.Tensor, group_offs: torch.Tensor, trans_a: bool,
                                 trans_b: bool, trans_c: bool, num_cu: Optional[int], default_backend: int,
                                 maybe_pre_sync: bool = False, schedule: str = "static") -> torch.Tensor:
    return _gg16.grouped_gemm_variable_k_impl(a, b, group_lens, group_offs, trans_a, trans_b, trans_c, num_cu, default_backend, schedule)


@grouped_gemm_variable_k_impl.register_fake
def _(a, b, group_lens, group_offs, trans_a, trans_b, trans_c, num_cu, default_backend, maybe_pre_sync=False, schedule="static"):
    return _variable_k_out(a, b, trans_a, trans_c, group_lens, a.dtype, True)


@_op("primus_turbo::grouped_gemm_variable_k_accum_impl", mutates_args={"out"}, device_types="cuda")
def grouped_gemm_variable_k_accum_impl(a: torch.Tensor, b: torch.Tensor, group_lens: torch.Tensor, group_offs: torch.Tensor, trans_a: bool,
                                       trans_b: bool, trans_c: bool, num_cu: Optional[int], default_backend: int, out: torch.Tensor,
                                       maybe_pre_sync: bool = False, schedule: str = "static") -> None:
    _gg16.grouped_gemm_variable_k_accum_impl(a, b, group_lens, group_offs, trans_a, trans_b, trans_c, num_cu, default_backend, out, schedule)


@grouped_gemm_variable_k_accum_impl.register_fake
def _(a, b, group_lens, group_offs, trans_a, trans_b, trans_c, num_cu, default_backend, out, maybe_pre_sync=False, schedule="static"):
    return None


# ------------------------------------------------------------------------------------------------ blockwise quantizers
@_op("primus_turbo::quant_fp8_blockwise_impl", mutates_args=(), device_types="cuda")
def quant_fp8_blockwise_impl(x: torch.Tensor, dtype: torch.dtype, axis: int, block_size: int = 128) -> Tuple[torch.Tensor, torch.Tensor]:
    return _q.quant_fp8_blockwise_impl(x, dtype, axis, block_size)


@quant_fp8_blockwise_impl.register_fake
def _(x, dtype, axis, block_size=128):
    M, N = x.shape
    s_shape = (M, _ceil_div(N, block_size)) if axis % 2 == 1 else (_ceil_div(M, block_size), N)
    return torch.empty((M, N), dtype=dtype, device=x.device), torch.empty(s_shape, dtype=torch.float32, device=x.device)


@_op("primus_turbo::dequant_fp8_blockwise_impl", mutates_args=(), device_types="cuda")
def dequant_fp8_blockwise_impl(x_fp8: torch.Tensor, scale_inv: torch.Tensor, out_dtype: torch.dtype, axis: int,
                               block_size: int = 128) -> torch.Tensor:
    return _q.dequant_fp8_blockwise_impl(x_fp8, scale_inv, out_dtype, axis, block_size)


@dequant_fp8_blockwise_impl.register_fake
def _(x_fp8, scale_inv, out_dtype, axis, block_size=128):
    return torch.empty(x_fp8.shape, dtype=out_dtype, device=x_fp8.device)


@_op("primus_turbo::dequant_fp8_blockwise_for_weight_impl", mutates_args=(), device_types="cuda")
def dequant_fp8_blockwise_for_weight_impl(w_fp8: torch.Tensor, scale_inv: torch.Tensor, out_dtype: torch.dtype,
                                          block_size: int = 128) -> torch.Tensor:
    return _q.dequant_fp8_blockwise_for_weight_impl(w_fp8, scale_inv, out_dtype, block_size)


@dequant_fp8_blockwise_for_weight_impl.register_fake
def _(w_fp8, scale_inv, out_dtype, block_size=128):
    return torch.empty(w_fp8.shape, dtype=out_dtype, device=w_fp8.device)


@_op("primus_turbo::quant_fp8_blockwise_dual_impl", mutates_args=(), device_types="cuda")
def quant_fp8_blockwise_dual_impl(x: torch.Tensor, dtype: torch.dtype,
                                  block_size: int = 128) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
    return _q.quant_fp8_blockwise_dual_impl(x, dtype, block_size)


@quant_fp8_blockwise_dual_impl.register_fake
def _(x, dtype, block_size=128):
    M, N = x.shape
    e = lambda shape, dt: torch.empty(shape, dtype=dt, device=x.device)
    return (e((M, N), dtype), e((M, _ceil_div(N, block_size)), torch.float32), e((M, N), dtype),
            e((_ceil_div(M, block_size), N), torch.float32))


@_op("primus_turbo::quant_fp8_blockwise_for_weight_impl", mutates_args=(), device_types="cuda")
def quant_fp8_blockwise_for_weight_impl(w: torch.Tensor, dtype: torch.dtype, block_size: int = 128) -> Tuple[torch.Tensor, torch.Tensor]:
    return _q.quant_fp8_blockwise_for_weight_impl(w, dtype, block_size)


@quant_fp8_blockwise_for_weight_impl.register_fake
def _(w, dtype, block_size=128):
    M, N = w.shape[-2:]
    lead = tuple(w.shape[:-2])
    return (torch.empty(w.shape, dtype=dtype, device=w.device),
            torch.empty(lead + (_ceil_div(M, block_size), _ceil_div(N, block_size)), dtype=torch.float32, device=w.device))


@_op("primus_turbo::quant_fp8_blockwise_segment_m_row_col_impl", mutates_args=(), device_types="cuda")
def quant_fp8_blockwise_segment_m_row_col_impl(x: torch.Tensor, dtype: torch.dtype, block_size: int, group_lens: torch.Tensor,
                                               group_offs: torch.Tensor, gemm_other_dim: Optional[int] = None
                                               ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
    return _q.quant_fp8_blockwise_segment_m_row_col_impl(x, dtype, block_size, group_lens, group_offs, gemm_other_dim)


@quant_fp8_blockwise_segment_m_row_col_impl.register_fake
def _(x, dtype, block_size, group_lens, group_offs, gemm_other_dim=None):
    M, N = x.shape
    G = group_lens.shape[0]
    m_alloc = M + G * block_size
    e = lambda shape, dt: torch.empty(shape, dtype=dt, device=x.device)
    return (e((M, N), dtype), e((m_alloc, N), dtype), e((_ceil_div(N, block_size), M), torch.float32),
            e((m_alloc // block_size, N), torch.float32), e((G,), torch.int64), e((G + 1,), torch.int64))


# ------------------------------------------------------------------------------------------------ pre-shuffled layouts
# (torch.ops.primus_turbo_cpp_extension.shuffle_scale / shuffle_weight of the reference: csrc/pytorch/bindings_pytorch.cpp)
@_op("primus_turbo::shuffle_scale", mutates_args=(), device_types="cuda")
def shuffle_scale(scale: torch.Tensor, layout: List[int]) -> torch.Tensor:
    return _q.shuffle_scale_impl(scale, tuple(layout))


@shuffle_scale.register_fake
def _(scale, layout):
    M, N = scale.shape
    return torch.empty((_ceil_div(M, 256) * 256, _ceil_div(N, 8) * 8), dtype=scale.dtype, device=scale.device)


@_op("primus_turbo::shuffle_weight", mutates_args=(), device_types="cuda")
def shuffle_weight(weight: torch.Tensor, layout: List[int]) -> torch.Tensor:
    return _q.shuffle_weight_impl(weight, tuple(layout))


@shuffle_weight.register_fake
def _(weight, layout):
    return torch.empty_like(weight)


REGISTERED = [
    "gemm_fp8_impl", "gemm_fp8_accum_impl", "gemm_fp4_impl", "gemm_fp4_accum_impl", "gemm_impl", "gemm_accum_impl",
    "grouped_gemm_fp8_impl", "grouped_gemm_fp8_variable_k_impl", "grouped_gemm_fp8_variable_k_accum_impl",
    "grouped_gemm_fp4_impl", "grouped_gemm_fp4_variable_k_impl", "grouped_gemm_fp4_variable_k_accum_impl",
    "grouped_gemm_impl", "grouped_gemm_variable_k_impl", "grouped_gemm_variable_k_accum_impl",
    "quant_fp8_blockwise_impl", "dequant_fp8_blockwise_impl", "dequant_fp8_blockwise_for_weight_impl",
    "quant_fp8_blockwise_dual_impl", "quant_fp8_blockwise_for_weight_impl", "quant_fp8_blockwise_segment_m_row_col_impl",
    "shuffle_scale", "shuffle_weight",
]
