"""Continuous-batching scheduler thread: cleanup -> admit -> prefill -> decode.

Public surface as in ``astrai/inference/core/scheduler.py:16-212`` (``start/stop/add_task/
remove_task/get_stats``, STOP sentinel through stream callbacks, fatal errors drain every
task).  The loop itself is different: every running sequence advances on every decode step
regardless of its position (the reference only steps the largest group of equal positions and
re-prefills the others), prefill runs once per task, and a prompt that is fully served by the
prefix cache still recomputes its last page so that positions stay correct.
"""

from __future__ import annotations

import logging
import threading
import time
from typing import Any, Dict, List, Optional, Tuple

import torch

from .cache import KVCache
from .executor import Executor
from .task import STOP, Task, TaskManager, TaskStatus
from ...models.automodel import AutoModel  # noqa: F401  (the types of the constructor's arguments; callers patch them)
from ...tokenize import AutoTokenizer  # noqa: F401
from ...utils.trace import trace_range

log = logging.getLogger(__name__)


class InferenceScheduler:
    def __init__(self, model, tokenizer, max_batch_size: int = 16, max_seq_len: Optional[int] = None,
                 max_prompt_len: int = 2048, page_size: int = 64, device=None, dtype: Optional[torch.dtype] = None):
        config = model.config
        if max_seq_len is None:
            max_seq_len = getattr(config, "max_len", None)
        if max_seq_len is None:
            raise ValueError("max_seq_len must be provided either as argument or in model config (config.max_len)")
        self.max_seq_len = max_seq_len
        first = next(model.parameters())
        self.device = device or first.device
        self.dtype = dtype or first.dtype
        n_pages = (max_batch_size * (max_seq_len + page_size) + page_size - 1) // page_size
        head_dim = config.dim // config.n_heads
        v_dim = None
        if getattr(config, "attn_type", "gqa") == "mla":
            head_dim = config.qk_nope_head_dim + config.qk_rope_head_dim
        # a tensor-parallel model keeps only this rank's KV heads and brings its own executor class
        n_kv_heads = getattr(model, "kv_heads_local", config.n_kv_heads)
        self._page_cache = KVCache(config.n_layers, n_pages, page_size, n_kv_heads, head_dim, self.device,
                                   self.dtype, v_dim)
        self._task_mgr = TaskManager(tokenizer, max_batch_size, max_seq_len, max_prompt_len)
        executor_cls = getattr(model, "executor_cls", None) or Executor
        self._executor = executor_cls(model, tokenizer, self._page_cache, self.device, self.dtype,
                                      max_seq_len=max_seq_len)
        self._running = False
        self._fatal_error: Optional[Exception] = None
        self._stopped = False          # set by stop(): requests that arrive afterwards are closed at once
        self._loop_thread: Optional[threading.Thread] = None
        self._steps = 0
        self._decode_tokens = 0
        self._busy_s = 0.0

    # -- public ---------------------------------------------------------------------------------
    def add_task(self, prompt, **kwargs) -> str:
        if self._fatal_error is not None or self._stopped:
            # the loop is gone: close the stream at once instead of queueing a request nobody will serve
            callback = kwargs.get("stream_callback")
            if callback:
                callback(STOP)
            return "task_rejected"
        return self._task_mgr.add_task(prompt, **kwargs)

    def remove_task(self, task_id: str) -> None:
        """Withdraw a request (any thread): its stream is closed here, its pages are released by the
        scheduler thread."""
        task = self._task_mgr.cancel(task_id)
        if task is not None and task.status == TaskStatus.ABORTED:
            self._emit(task, STOP)

    def get_stats(self) -> Dict[str, Any]:
        stats = self._task_mgr.get_stats()
        stats.update(self._task_mgr.latency_stats())
        stats.update({"decode_steps": self._steps, "decode_tokens": self._decode_tokens,
                      "decode_tokens_per_s": self._decode_tokens / self._busy_s if self._busy_s > 0 else 0.0,
                      "free_pages": self._page_cache.free_pages(),
                      "decode_graphs": sum(1 for s in getattr(self._executor, "_slots", {}).values() if s.graph is not None)})
        return stats

    def get_histograms(self) -> Dict[str, Dict[str, Any]]:
        return self._task_mgr.histograms()

    def start(self) -> None:
        if self._running:
            return
        self._stopped = False
        self._running = True
        self._loop_thread = threading.Thread(target=self._run_generation_loop, daemon=True, name="kb200-scheduler")
        self._loop_thread.start()

    def stop(self) -> None:
        self._stopped = True
        self._running = False
        self._task_mgr.wake()
        if self._loop_thread is not None:
            self._loop_thread.join(timeout=5.0)
        self._drain()
        self._executor.close()
        if torch.cuda.is_available():
            torch.cuda.empty_cache()

    # -- loop -----------------------------------------------------------------------------------
    def _emit(self, task: Task, item) -> None:
        """Hand a token (or STOP) to the request's consumer.  A consumer that raises - an event loop
        that was closed, a broken pipe - costs that request only: it is aborted, the loop goes on."""
        if task.stream_callback is None:
            return
        try:
            task.stream_callback(item)
        except Exception as exc:
            log.warning("stream callback of %s failed (%s); the request is dropped", task.task_id, exc)
            task.stream_callback = None
            if task.status == TaskStatus.RUNNING:
                task.status = TaskStatus.ABORTED

    def _drain(self) -> None:
        for task in self._task_mgr.get_active_tasks():
            self._emit(task, STOP)
            self._page_cache.task_free(task.task_id)
        for task in self._task_mgr.get_waiting_tasks():
            self._emit(task, STOP)
        self._task_mgr.clear_queues()

    def _admit(self) -> None:
        room = self._task_mgr.max_batch_size - len(self._task_mgr.get_active_tasks())
        if room <= 0:
            return
        rejected: List[Task] = []
        for task in self._task_mgr.pull_candidates(room):
            if not rejected and self._page_cache.task_alloc(task.task_id, task.prompt_ids):
                task.prefilled = False
                self._task_mgr.activate(task)
            else:
                rejected.append(task)  # keep FIFO order: nothing overtakes a task that did not fit
        if rejected:
            self._task_mgr.return_to_waiting(rejected)

    def _accept(self, task: Task, token: int, stop_ids: List[int]) -> None:
        task.output_ids.append(token)
        task.output_tokens += 1
        if task.first_token_time is None:
            task.first_token_time = time.time()
        self._emit(task, self._task_mgr.tokenizer.decode([token]))
        if task.is_finished(stop_ids):
            # finished before the stream closes: the client's release of the task (which may arrive the moment
            # it sees STOP) must not turn a completed request into an aborted one in the statistics
            task.status = TaskStatus.FINISHED
            self._emit(task, STOP)

    HEALTH_EVERY = 64         # decode steps between two reads of the kernels' error word

    def _check_device(self) -> None:
        """A bounded wait that ran out inside a kernel leaves a code in the device's error word;
        surface it as an exception (the loop's fatal-error path then releases every request)."""
        if torch.device(self.device).type == "cuda":
            from ...ops import raise_on_device_error

            raise_on_device_error()

    PAD_BUCKET = 256          # prompts whose lengths fall into the same bucket are prefilled together
    PAD_BATCH_TOKENS = 32768  # padded tokens per prefill batch at most

    def _prefill(self, stop_ids: List[int]) -> None:
        page = self._page_cache.page_size
        groups: Dict[Tuple[int, int], List[Task]] = {}
        padded: Dict[int, List[Task]] = {}
        for t in self._task_mgr.get_active_tasks():
            if getattr(t, "prefilled", False) or t.status != TaskStatus.RUNNING:
                continue
            n = len(t.prompt_ids)
            cached = min(self._page_cache.task_cached(t.task_id), ((n - 1) // page) * page)
            t.input_tokens = n
            if cached == 0:   # nothing from the prefix cache: can share a right-padded batch
                padded.setdefault((n + self.PAD_BUCKET - 1) // self.PAD_BUCKET, []).append(t)
            else:
                groups.setdefault((n, cached), []).append(t)

        def done(group, first, cached):
            for t, tok in zip(group, first):
                t.prefilled = True
                self._page_cache.task_record_hashes(t.task_id, t.prompt_ids, start_logical_page=cached // page)
                self._accept(t, tok, stop_ids)

        for (n, cached), group in groups.items():
            with trace_range("prefill"):
                first = self._executor.execute_prefill(group, n, cached)
            done(group, first, cached)
        for bucket, tasks in padded.items():
            per_batch = max(1, self.PAD_BATCH_TOKENS // (bucket * self.PAD_BUCKET))
            for i in range(0, len(tasks), per_batch):
                group = tasks[i:i + per_batch]
                if len({len(t.prompt_ids) for t in group}) == 1:
                    first = self._executor.execute_prefill(group, len(group[0].prompt_ids), 0)
                else:
                    first = self._executor.execute_prefill_padded(group)
                done(group, first, 0)

    def _decode(self, stop_ids: List[int]) -> None:
        ready: List[Task] = []
        for t in self._task_mgr.get_active_tasks():
            if not getattr(t, "prefilled", False) or t.status != TaskStatus.RUNNING or t.is_finished(stop_ids):
                continue
            if self._page_cache.task_extend(t.task_id, t.next_pos - 1):
                ready.append(t)
            else:  # out of pages: give up on this sequence, free its memory next iteration
                t.status = TaskStatus.ABORTED
                self._emit(t, STOP)
        if not ready:
            return
        t0 = time.perf_counter()
        with trace_range("decode_step"):
            tokens = self._executor.execute_decode(ready)
        self._busy_s += time.perf_counter() - t0
        self._steps += 1
        if self._steps % self.HEALTH_EVERY == 0:
            self._check_device()
        self._decode_tokens += len(ready)
        for t, tok in zip(ready, tokens):
            self._accept(t, tok, stop_ids)

    def _run_generation_loop(self) -> None:
        stop_ids = list(self._task_mgr.tokenizer.stop_ids)
        try:
            while self._running:
                for task in self._task_mgr.remove_finished_tasks(stop_ids):
                    self._page_cache.task_free(task.task_id)
                self._admit()
                if not self._task_mgr.has_work():
                    self._task_mgr.wait_for_tasks(timeout=1.0)
                    continue
                self._prefill(stop_ids)
                self._decode(stop_ids)
        except Exception as exc:  # fatal: release everything that is waiting on us
            self._fatal_error = exc
            self._running = False
            log.error("Scheduler loop crashed: %s", exc, exc_info=True)
            self._drain()
