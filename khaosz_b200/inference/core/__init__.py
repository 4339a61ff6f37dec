from .cache import Allocator, KVCache, KvcacheView, PagePool, PrefixCache, Storage, TaskTable, page_hash
from .executor import Executor
from .scheduler import InferenceScheduler
from .task import STOP, Task, TaskManager, TaskStatus

__all__ = ["Allocator", "KVCache", "KvcacheView", "PagePool", "PrefixCache", "Storage", "TaskTable", "page_hash",
           "Executor", "InferenceScheduler", "STOP", "Task", "TaskManager", "TaskStatus"]
