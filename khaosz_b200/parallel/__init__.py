from .executor import (AccumOptimizer, AccumScheduler, BaseExecutor, DDPExecutor, ExecutorFactory, FSDPExecutor,
                       FullShardExecutor, GradientState, NoneExecutor, TPExecutor)
from .fsdp_model import FullShardLM, full_shard
from .setup import (get_current_device, get_rank, get_world_size, only_on_rank, setup_parallel, spawn_parallel_fn)
from .tensor_parallel import ColumnParallelLinear, RowParallelLinear
from .tp_model import TensorParallelLM, tensorize

__all__ = ["AccumOptimizer", "AccumScheduler", "BaseExecutor", "DDPExecutor", "ExecutorFactory", "FSDPExecutor",
           "FullShardExecutor", "GradientState", "NoneExecutor", "TPExecutor", "FullShardLM", "full_shard",
           "get_current_device", "get_rank", "get_world_size", "only_on_rank", "setup_parallel", "spawn_parallel_fn",
           "ColumnParallelLinear", "RowParallelLinear", "TensorParallelLM", "tensorize"]
