from .grouped_linear import *  # noqa: F401,F403
from .grouped_linear_lowp import *  # noqa: F401,F403
from .linear_fp8 import *  # noqa: F401,F403
from ._weight_cache import invalidate_on_optimizer_step, invalidate_quantized_weight_caches  # noqa: F401
