"""Continuous-batching inference: ``core`` (paged KV cache, tasks, executor, scheduler),
``engine`` (facade), ``sample`` (sampling strategies + fused kernel), ``api`` (HTTP)."""

from .core import (STOP, Allocator, Executor, InferenceScheduler, KVCache, KvcacheView, PagePool, PrefixCache,
                   Storage, Task, TaskManager, TaskStatus, TaskTable, page_hash)
from .engine import GenerateResult, GenerationRequest, InferenceEngine
from .sample import (BaseSamplingStrategy, SamplingPipeline, TemperatureStrategy, TopKStrategy, TopPStrategy, sample)

__all__ = ["STOP", "Allocator", "Executor", "InferenceScheduler", "KVCache", "KvcacheView", "PagePool", "PrefixCache",
           "Storage", "Task", "TaskManager", "TaskStatus", "TaskTable", "page_hash", "GenerateResult",
           "GenerationRequest", "InferenceEngine", "BaseSamplingStrategy", "SamplingPipeline", "TemperatureStrategy",
           "TopKStrategy", "TopPStrategy", "sample"]
