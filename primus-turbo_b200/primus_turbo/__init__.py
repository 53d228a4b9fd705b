"""B200-native drop-in for the low-precision GEMM path of Primus-Turbo.

Only `primus_turbo.pytorch` (quantize / dequantize, gemm_fp8 / gemm_fp4, grouped_gemm_fp8 /
grouped_gemm_fp4 and the types they take) is provided.  All device work is done by the CUDA
library libpt_b200.so through its C ABI (include/pt_b200.h); there is no other code path.
"""
__version__ = "0.1.0"
