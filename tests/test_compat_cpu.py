"""Import compatibility with code written against the reference: back-end manager, logger, environment names, and the
torch.library registrations with their fake implementations (no GPU needed: fake tensors carry a CUDA device)."""
import logging

import pytest
import torch


def test_backend_manager_accepts_and_ignores():
    from primus_turbo.pytorch.core.backend import BackendChoice, BackendType, GlobalBackendManager, PrecisionType
    assert [m.name for m in BackendType][:8] == ["CK", "HIPBLASLT", "AITER", "TRITON", "DEEP_EP", "TURBO", "FLYDSL", "HIPKITTENS"]
    assert BackendType.HIPBLASLT.value == 2      # the ints that travel through `default_backend`
    GlobalBackendManager.reset()
    assert GlobalBackendManager.get_gemm_backend(PrecisionType.FP8) is None
    GlobalBackendManager.set_gemm_backend(BackendType.HIPBLASLT)
    assert GlobalBackendManager.get_gemm_backend(PrecisionType.FP8) == BackendChoice(BackendType.HIPBLASLT)
    GlobalBackendManager.set_grouped_gemm_backend(BackendType.TRITON, PrecisionType.FP4)
    assert GlobalBackendManager.get_grouped_gemm_backend(PrecisionType.FP4).backend == BackendType.TRITON
    assert GlobalBackendManager.get_grouped_gemm_backend(PrecisionType.FP8) is None
    GlobalBackendManager.set_auto_tune(False)
    assert GlobalBackendManager.auto_tune_enabled() is False
    GlobalBackendManager.reset()
    assert GlobalBackendManager.get_gemm_backend(PrecisionType.FP8) is None


def test_backend_env_grammar(monkeypatch):
    from primus_turbo.common.constants import ENV_GEMM_BACKEND
    from primus_turbo.pytorch.core.backend import BackendType, GlobalBackendManager, PrecisionType
    GlobalBackendManager.reset()
    monkeypatch.setenv(ENV_GEMM_BACKEND, "FP8:triton,other:hipblaslt")
    assert GlobalBackendManager.get_gemm_backend(PrecisionType.FP8).backend == BackendType.TRITON
    assert GlobalBackendManager.get_gemm_backend(PrecisionType.FP4).backend == BackendType.HIPBLASLT
    monkeypatch.setenv(ENV_GEMM_BACKEND, "autotune")
    assert GlobalBackendManager.get_gemm_backend(PrecisionType.FP8).auto_tune
    monkeypatch.setenv(ENV_GEMM_BACKEND, "no_such_backend")
    assert GlobalBackendManager.get_gemm_backend(PrecisionType.FP8) is None


def test_logger_once_and_levels():
    from primus_turbo.common.logger import LogLevelEnum, logger
    assert str(LogLevelEnum.INFO) == "INFO"
    seen = []

    class _Collect(logging.Handler):
        def emit(self, record):
            seen.append(record.getMessage())

    lg = logging.getLogger("primus_turbo")
    h = _Collect()
    lg.addHandler(h)
    try:
        logger.set_level("INFO")
        for _ in range(3):
            logger.info("only once", once=True)
        logger.info("rank 7 only", rank=7)
        logger.debug("below the level")
        logger.warning("every time")
        logger.warning("every time")
        assert seen.count("only once") == 1 and seen.count("every time") == 2
        assert "rank 7 only" not in seen and "below the level" not in seen
    finally:
        lg.removeHandler(h)
        logger.set_level("WARNING")


def test_names_the_reference_operators_import():
    """Every name primus_turbo/pytorch/ops/gemm_fp8.py of the reference imports from the package resolves here."""
    from primus_turbo.pytorch.core.backend import BackendType  # noqa: F401
    from primus_turbo.pytorch.core.low_precision import (Float8QuantConfig, Format, ScaleDtype,  # noqa: F401
                                                         ScalingGranularity, ScalingRecipe)
    from primus_turbo.pytorch.core.quantized_tensor import (QuantizedTensor, QuantizedTensorPair,  # noqa: F401
                                                            check_quantized_tensor)
    from primus_turbo.pytorch.kernels.gemm.gemm_fp8_impl import gemm_fp8_accum_impl, gemm_fp8_impl  # noqa: F401
    from primus_turbo.pytorch.kernels.quantization.quantization_impl import (quant_fp8_blockwise_impl,  # noqa: F401
                                                                             quantize_mxfp8_impl)
    from primus_turbo.pytorch.ops.quantization import quantize_fp8, quantize_fp8_with_trans  # noqa: F401
    from primus_turbo.pytorch.ops.utils import _get_dummy_wgrad, _get_fp8_dtype, _setup_fused_grad_accum  # noqa: F401


def test_custom_ops_are_registered_with_fake_impls():
    from torch._subclasses.fake_tensor import FakeTensorMode

    from primus_turbo.pytorch.kernels import registry
    for name in registry.REGISTERED:
        assert hasattr(torch.ops.primus_turbo, name), name
    f8 = torch.float8_e4m3fn
    with FakeTensorMode():
        e = lambda shape, dt=torch.bfloat16: torch.empty(shape, dtype=dt, device="cuda")
        a, b = e((256, 512), f8), e((384, 512), f8)
        sa, sb = e((), torch.float32), e((), torch.float32)
        c = torch.ops.primus_turbo.gemm_fp8_impl(a, sa, False, b, sb, True, torch.bfloat16, False, 1, 2)
        assert tuple(c.shape) == (256, 384) and c.dtype == torch.bfloat16 and c.device.type == "cuda"
        ct = torch.ops.primus_turbo.gemm_fp8_impl(a, sa, False, b, sb, True, torch.float16, True, 1, 2)
        assert tuple(ct.shape) == (384, 256)
        q, s = torch.ops.primus_turbo.quant_fp8_blockwise_impl(e((300, 520)), f8, 1)
        assert tuple(q.shape) == (300, 520) and tuple(s.shape) == (300, 5) and s.dtype == torch.float32
        q, s = torch.ops.primus_turbo.quant_fp8_blockwise_impl(e((300, 520)), f8, 0)
        assert tuple(s.shape) == (3, 520)
        qr, sr, qc, sc = torch.ops.primus_turbo.quant_fp8_blockwise_dual_impl(e((256, 384)), f8)
        assert tuple(sr.shape) == (256, 3) and tuple(sc.shape) == (2, 384)
        sh = torch.ops.primus_turbo.shuffle_scale(e((100, 9), torch.float8_e8m0fnu), [16, 16])
        assert tuple(sh.shape) == (256, 16) and sh.dtype == torch.float8_e8m0fnu
        assert tuple(torch.ops.primus_turbo.shuffle_weight(e((32, 64), torch.uint8), [16, 16]).shape) == (32, 64)
        qw, sw = torch.ops.primus_turbo.quant_fp8_blockwise_for_weight_impl(e((4, 256, 384)), f8)
        assert tuple(sw.shape) == (4, 2, 3)
        lens, offs = e((4,), torch.int64), e((5,), torch.int64)
        outs = torch.ops.primus_turbo.quant_fp8_blockwise_segment_m_row_col_impl(e((1000, 256)), f8, 128, lens, offs)
        assert tuple(outs[1].shape) == (1000 + 4 * 128, 256) and tuple(outs[2].shape) == (2, 1000) and tuple(outs[5].shape) == (5,)
        y = torch.ops.primus_turbo.grouped_gemm_fp8_impl(e((1000, 256), f8), e((4, 512, 256), f8), e((2, 1000), torch.float32),
                                                         e((4, 4, 2), torch.float32), lens, offs, False, True, torch.bfloat16, 3, None, 2)
        assert tuple(y.shape) == (1000, 512)
        dw = torch.ops.primus_turbo.grouped_gemm_fp8_variable_k_impl(e((1512, 256), f8), e((1512, 512), f8), e((12, 256), torch.float32),
                                                                     e((12, 512), torch.float32), lens, offs, True, False, True,
                                                                     torch.bfloat16, 3, None, 2)
        assert tuple(dw.shape) == (4, 512, 256)
        g = torch.ops.primus_turbo.gemm_impl(e((64, 128)), False, e((128, 96)), False, torch.bfloat16, False, 2)
        assert tuple(g.shape) == (64, 96)
        gg = torch.ops.primus_turbo.grouped_gemm_impl(e((1000, 256)), e((4, 512, 256)), lens, offs, False, True, None, 2)
        assert tuple(gg.shape) == (1000, 512)
