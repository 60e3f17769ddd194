from .bootstrap import init_distributed, shutdown, ProcessMesh, barrier, get_rank, world_size, is_main_process
from .zero import ShardedEngine, Bucket
