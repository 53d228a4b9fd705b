"""primus_turbo.pytorch: the operator surface of the low-precision GEMM path."""
from .. import _clib

_clib.load()  # fail at import, loudly, when the CUDA library is absent

from . import modules, ops  # noqa: E402,F401
from .kernels import registry  # noqa: E402,F401  (torch.ops.primus_turbo.* with fake implementations)
from .core.low_precision import float4_e2m1fn_x2, float8_e4m3, float8_e5m2  # noqa: E402,F401
