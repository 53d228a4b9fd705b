from .grouped_linear import *  # noqa: F401,F403
from .grouped_linear_lowp import *  # noqa: F401,F403
from .linear_fp8 import *  # noqa: F401,F403
