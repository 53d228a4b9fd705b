"""Names of the environment variables the library reads, in one place.

The first group keeps the reference's names (primus_turbo/common/constants.py) so that launch scripts written for it keep
working: the back-end selectors are read and validated but select nothing, because this build has a single back end per
operator.  The second group are this build's own switches.
"""
# logger level: DEBUG / INFO / WARNING / ERROR / CRITICAL (default WARNING)
ENV_LOG_LEVEL = "PRIMUS_TURBO_LOG_LEVEL"
# accepted for compatibility; there is one GEMM / grouped-GEMM back end here
ENV_GEMM_BACKEND = "PRIMUS_TURBO_GEMM_BACKEND"
ENV_GROUPED_GEMM_BACKEND = "PRIMUS_TURBO_GROUPED_GEMM_BACKEND"
ENV_MOE_DISPATCH_COMBINE_BACKEND = "PRIMUS_TURBO_MOE_DISPATCH_COMBINE_BACKEND"
ENV_ATTN_BACKEND = "PRIMUS_TURBO_ATTN_BACKEND"
ENV_SPARSE_ATTN_BACKEND = "PRIMUS_TURBO_SPARSE_ATTN_BACKEND"
ENV_AUTO_TUNE = "PRIMUS_TURBO_AUTO_TUNE"

# ---- switches of the B200 library (read by the CUDA library or the Python glue at call time)
ENV_PT_NO_PDL = "PT_NO_PDL"                          # launch without programmatic stream serialization
ENV_PT_GEMM_PAIR = "PT_GEMM_PAIR"                    # 0: single-CTA GEMM tiles everywhere
ENV_PT_BW_GEMM_PAIR = "PT_BW_GEMM_PAIR"              # 1: CTA-pair form of the block-scaled GEMM
ENV_PT_MX_QUANT_NO_TMA = "PT_MX_QUANT_NO_TMA"        # MX quantizer: one-CTA-per-tile kernel
ENV_PT_MX_QUANT_NO_SPLIT = "PT_MX_QUANT_NO_SPLIT"    # MX quantizer: single-role consumer warps instead of the warp-split kernel
ENV_PT_CHECK_STATUS = "PT_CHECK_STATUS"              # 1: read the kernels' status word after every GEMM call (synchronises)
