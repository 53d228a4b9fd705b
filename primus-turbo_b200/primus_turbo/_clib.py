"""ctypes binding of libpt_b200.so (C ABI declared in include/pt_b200.h).

The library is the only implementation of every operator in this package: when it cannot be
loaded the import fails with instructions to build it, and no operator falls back to anything.
"""
import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "lib", "libpt_b200.so")

c_void_p, c_int, c_int64, c_float, c_size_t, c_uint = (ctypes.c_void_p, ctypes.c_int, ctypes.c_int64, ctypes.c_float,
                                                       ctypes.c_size_t, ctypes.c_uint)

# name -> (restype, argtypes); mirrors include/pt_b200.h one to one
SIGNATURES = {
    "pt_last_error": (ctypes.c_char_p, []),
    "pt_device_sm_count": (c_int, []),
    "pt_set_default_status": (c_int, [c_void_p]),
    "pt_wait_probe": (c_int, [c_int64, c_void_p, c_void_p, c_void_p]),
    "pt_quantize_fp8_tensorwise_workspace_bytes": (c_size_t, []),
    "pt_quantize_fp8_tensorwise": (c_int, [c_void_p, c_int, c_int64, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
                                           c_size_t, c_void_p]),
    "pt_quantize_fp8_rowwise": (c_int, [c_void_p, c_int, c_int64, c_int64, c_int64, c_int, c_int, c_void_p, c_void_p,
                                        c_void_p, c_void_p, c_size_t, c_void_p]),
    "pt_quantize_fp8_colscale_noalloc": (c_int, [c_void_p, c_int, c_int64, c_int64, c_int64, c_int, c_void_p, c_void_p,
                                                 c_void_p]),
    "pt_dequantize_fp8": (c_int, [c_void_p, c_int, c_void_p, c_int, c_int64, c_int64, c_int64, c_void_p, c_int, c_void_p]),
    "pt_quantize_fp8_blockwise": (c_int, [c_void_p, c_int, c_int64, c_int64, c_int, c_void_p, c_void_p, c_void_p,
                                          c_void_p, c_void_p]),
    "pt_quantize_fp8_blockwise_weight": (c_int, [c_void_p, c_int, c_int64, c_int64, c_int64, c_int, c_void_p, c_void_p,
                                                 c_void_p]),
    "pt_quantize_fp8_blockwise_segment_m": (c_int, [c_void_p, c_int, c_int64, c_int64, c_int, c_void_p, c_void_p, c_int,
                                                    c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]),
    "pt_dequantize_fp8_blockwise": (c_int, [c_void_p, c_int, c_void_p, c_int, c_int64, c_int64, c_int64, c_void_p, c_int,
                                            c_void_p]),
    "pt_compute_group_offs": (c_int, [c_void_p, c_int, c_void_p, c_void_p]),
    "pt_compute_padded_group_offs": (c_int, [c_void_p, c_int, c_int64, c_void_p, c_void_p, c_void_p]),
    "pt_quantize_mx": (c_int, [c_void_p, c_int, c_int64, c_int64, c_int64, c_int, c_uint, c_void_p, c_void_p, c_void_p,
                               c_void_p, c_void_p]),
    "pt_grouped_quantize_mx": (c_int, [c_void_p, c_int, c_int64, c_int64, c_int, c_void_p, c_void_p, c_void_p, c_int, c_uint,
                                       c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_void_p]),
    "pt_dequantize_mx": (c_int, [c_void_p, c_int, c_void_p, c_int64, c_int64, c_int64, c_int, c_void_p, c_int, c_void_p]),
    "pt_moe_row_id_map_workspace_bytes": (c_size_t, [c_int64, c_int]),
    "pt_moe_make_row_id_map": (c_int, [c_void_p, c_int, c_int64, c_int, c_void_p, c_void_p, c_void_p, c_size_t, c_void_p]),
    "pt_moe_permute": (c_int, [c_void_p, c_int64, c_int64, c_int, c_void_p, c_void_p, c_int, c_int64, c_void_p, c_void_p, c_void_p]),
    "pt_moe_unpermute": (c_int, [c_void_p, c_int, c_int64, c_int64, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p]),
    "pt_moe_unpermute_bwd_with_probs": (c_int, [c_void_p, c_void_p, c_int, c_int64, c_int64, c_int, c_void_p, c_void_p, c_int, c_void_p,
                                                c_void_p, c_void_p]),
    "pt_glu_quantize_mx_row": (c_int, [c_void_p, c_int, c_void_p, c_void_p, c_int64, c_int64, c_int, c_int, c_void_p, c_void_p, c_void_p]),
    "pt_rmsnorm_quantize_mx_row": (c_int, [c_void_p, c_int, c_void_p, c_float, c_int, c_int64, c_int64, c_int, c_void_p, c_void_p, c_void_p,
                                           c_void_p]),
    "pt_shuffle_e8m0_scale": (c_int, [c_void_p, c_int64, c_int64, c_void_p, c_void_p]),
    "pt_shuffle_mx_codes": (c_int, [c_void_p, c_int64, c_int64, c_void_p, c_void_p]),
    "pt_glu_fwd": (c_int, [c_void_p, c_int, c_void_p, c_void_p, c_int64, c_int64, c_int, c_void_p, c_void_p]),
    "pt_glu_bwd": (c_int, [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int64, c_int64, c_int, c_void_p, c_void_p, c_void_p]),
    "pt_rmsnorm_fwd": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_float, c_int, c_int64, c_int64, c_void_p, c_void_p, c_void_p, c_void_p]),
    "pt_rmsnorm_bwd_parts": (c_int, [c_int64]),
    "pt_rmsnorm_bwd": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int64, c_int64, c_void_p, c_void_p, c_void_p,
                               c_int, c_void_p]),
    "pt_glu_quantize_mx": (c_int, [c_void_p, c_int, c_void_p, c_void_p, c_int64, c_int64, c_int, c_int, c_uint, c_void_p, c_void_p, c_void_p,
                                   c_void_p, c_void_p]),
    "pt_grouped_glu_quantize_mx": (c_int, [c_void_p, c_int, c_void_p, c_void_p, c_int64, c_int64, c_int, c_int, c_void_p, c_void_p, c_void_p,
                                           c_int, c_uint, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_void_p]),
    "pt_rmsnorm_quantize_mx": (c_int, [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int64, c_int64, c_int, c_uint, c_void_p, c_void_p, c_void_p,
                                       c_void_p, c_void_p]),
    "pt_transpose_2d": (c_int, [c_void_p, c_int64, c_int64, c_int, c_void_p, c_void_p]),
    "pt_transpose_batched": (c_int, [c_void_p, c_int64, c_int64, c_int64, c_int, c_void_p, c_void_p]),
    "pt_grouped_transpose_pad": (c_int, [c_void_p, c_int64, c_int64, c_int, c_void_p, c_void_p, c_int, c_void_p, c_int64, c_void_p]),
    "pt_zero_rows_from": (c_int, [c_void_p, c_int64, c_int64, c_void_p, c_void_p]),
    "pt_gemm": (c_int, [c_void_p, c_void_p, c_int, c_void_p, c_int, c_int64, c_int64, c_int64, c_float, c_void_p, c_void_p]),
    "pt_grouped_gemm": (c_int, [c_void_p, c_void_p, c_int, c_void_p, c_int, c_int64, c_int64, c_int64, c_void_p, c_int, c_float,
                                c_int, c_void_p, c_void_p]),
    "pt_grouped_gemm_variable_k": (c_int, [c_void_p, c_void_p, c_int, c_void_p, c_int, c_int64, c_int64, c_int64, c_void_p, c_int,
                                           c_float, c_int, c_void_p, c_void_p]),
    "pt_gemm_fp8_mn": (c_int, [c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p, c_int, c_int, c_void_p, c_int, c_int, c_int64, c_int64,
                               c_int64, c_float, c_void_p, c_void_p]),
    "pt_gemm_fp8": (c_int, [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int64,
                            c_int64, c_int64, c_float, c_int, c_void_p, c_size_t, c_void_p, c_void_p]),
    "pt_gemm_fp8_workspace_bytes": (c_size_t, [c_int, c_int64, c_int64, c_int64, c_int, c_int, c_int]),
    "pt_grouped_gemm_fp8": (c_int, [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int,
                                    c_int64, c_int64, c_int64, c_int64, c_void_p, c_void_p, c_int, c_float, c_int, c_int,
                                    c_void_p, c_size_t, c_void_p, c_void_p]),
    "pt_gemm_fp4": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int64, c_int64, c_int64, c_float, c_int,
                            c_void_p, c_size_t, c_void_p, c_void_p]),
    "pt_grouped_gemm_fp4": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int64, c_int64, c_int64, c_int64,
                                    c_void_p, c_void_p, c_int, c_float, c_int, c_int, c_void_p, c_size_t, c_void_p, c_void_p]),
    "pt_grouped_gemm_fp4_variable_k": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int64, c_int64, c_int64,
                                               c_void_p, c_int, c_float, c_int, c_int, c_void_p, c_size_t, c_void_p, c_void_p]),
    "pt_gemm_fp4_workspace_bytes": (c_size_t, [c_int64, c_int64, c_int64, c_int, c_int, c_int]),
    "pt_grouped_gemm_fp8_variable_k": (c_int, [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int,
                                               c_int64, c_int64, c_int64, c_void_p, c_int, c_float, c_int, c_int, c_void_p,
                                               c_size_t, c_void_p, c_void_p]),
    "pt_grouped_gemm_fp8_blockwise": (c_int, [c_void_p, c_int, c_int, c_int64, c_int64, c_void_p, c_int, c_int64, c_int64,
                                              c_void_p, c_int, c_int, c_int64, c_int64, c_void_p, c_int, c_int64, c_int64,
                                              c_int64, c_void_p, c_int, c_int64, c_int64, c_int64, c_void_p, c_void_p,
                                              c_void_p, c_int, c_float, c_int, c_void_p, c_void_p]),
}

_lib = None


def load():
    """Loads the CUDA library once and attaches the signatures; raises if it is missing."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python primus-turbo_b200/build.py` "
            "(nvcc, sm_100a). This package has no other implementation of its operators.")
    lib = ctypes.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError here means header and library are out of step
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def check(rc: int, what: str = ""):
    if rc != 0:
        msg = load().pt_last_error().decode("utf-8", "replace")
        raise RuntimeError(f"{what or 'libpt_b200'} failed ({rc}): {msg}")
