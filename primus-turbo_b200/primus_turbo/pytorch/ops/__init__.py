from .gemm import *  # noqa: F401,F403
from .gemm_fp4 import *  # noqa: F401,F403
from .gemm_fp8 import *  # noqa: F401,F403
from .grouped_gemm import *  # noqa: F401,F403
from .grouped_gemm_fp4 import *  # noqa: F401,F403
from .grouped_gemm_fp8 import *  # noqa: F401,F403
from .quantization import *  # noqa: F401,F403
from .moe import *  # noqa: F401,F403
