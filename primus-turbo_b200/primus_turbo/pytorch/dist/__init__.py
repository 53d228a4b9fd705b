from .partitioner import ColumnShardedLinear, ExpertShardedGroupedLinear, column_shard, expert_shard  # noqa: F401
