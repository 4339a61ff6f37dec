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


# The HTTP layer's names are part of this package's surface too, as in the reference
# (``astrai/inference/__init__.py``); they resolve on first use so that importing the engine does not
# import FastAPI.
_API_NAMES = ("AnthropicMessage", "ChatCompletionRequest", "ChatMessage", "GenContext", "MessagesRequest",
              "ProtocolHandler", "StopChecker", "StopInfo", "app", "run_server", "AnthropicResponseBuilder",
              "OpenAIResponseBuilder", "ResponseBuilder")
__all__ += list(_API_NAMES)


def __getattr__(name):
    if name in _API_NAMES:
        from . import api

        return getattr(api, name)
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
