from .executor import (AccumOptimizer, AccumScheduler, BaseExecutor, DDPExecutor, ExecutorFactory, FSDPExecutor,
                       GradientState, NoneExecutor)
from .setup import (get_current_device, get_rank, get_world_size, only_on_rank, setup_parallel, spawn_parallel_fn)

__all__ = ["AccumOptimizer", "AccumScheduler", "BaseExecutor", "DDPExecutor", "ExecutorFactory", "FSDPExecutor",
           "GradientState", "NoneExecutor", "get_current_device", "get_rank", "get_world_size", "only_on_rank",
           "setup_parallel", "spawn_parallel_fn"]
