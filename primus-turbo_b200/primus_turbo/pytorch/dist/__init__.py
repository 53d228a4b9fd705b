from .partitioner import ColumnShardedLinear, ExpertShardedGroupedLinear, column_shard, expert_shard  # noqa: F401
from .fp8_alltoall import FP8AllToAll  # noqa: F401
