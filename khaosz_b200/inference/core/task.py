"""Generation tasks and the thread-safe queues the scheduler pulls from
(reference: ``astrai/inference/core/task.py:13-209``).  Tasks additionally record
time-to-first-token and finish time so the engine can report latency statistics."""

from __future__ import annotations

import bisect
import threading
import time
import uuid
from collections import deque
from enum import Enum
from typing import Any, Callable, Deque, Dict, List, Optional

STOP = object()  # sentinel pushed through stream callbacks when a task ends

LATENCY_BUCKETS_S = (0.005, 0.01, 0.025, 0.05, 0.1, 0.25, 0.5, 1.0, 2.5, 5.0, 10.0, 30.0, 60.0, 120.0, 300.0)
RECENT = 65536   # finished requests kept for the percentile figures


class Histogram:
    """Cumulative histogram over fixed upper bounds (the shape a Prometheus scrape expects)."""

    def __init__(self, bounds=LATENCY_BUCKETS_S):
        self.bounds = tuple(bounds)
        self.counts = [0] * (len(self.bounds) + 1)   # last slot: above every bound
        self.total = 0.0
        self.n = 0

    def observe(self, value: float) -> None:
        self.counts[bisect.bisect_left(self.bounds, value)] += 1
        self.total += value
        self.n += 1

    def snapshot(self) -> Dict[str, Any]:
        running, cumulative = 0, []
        for c in self.counts[:-1]:
            running += c
            cumulative.append(running)
        return {"bounds": list(self.bounds), "cumulative": cumulative, "count": self.n, "sum": self.total}


class TaskStatus(Enum):
    PENDING = "pending"
    RUNNING = "running"
    FINISHED = "finished"
    ABORTED = "aborted"


class Task:
    def __init__(self, task_id: str, prompt_ids: List[int], max_tokens: Optional[int] = None, temperature: float = 1.0,
                 top_p: float = 1.0, top_k: int = 50, stream_callback: Optional[Callable] = None):
        self.task_id, self.prompt_ids, self.max_tokens = task_id, prompt_ids, max_tokens
        self.temperature, self.top_p, self.top_k = temperature, top_p, top_k
        self.status = TaskStatus.PENDING
        self.output_ids: List[int] = []
        self.input_tokens = 0
        self.output_tokens = 0
        self.arrival_time = time.time()
        self.first_token_time: Optional[float] = None
        self.finish_time: Optional[float] = None
        self.stream_callback = stream_callback

    @property
    def next_pos(self) -> int:
        return self.input_tokens + len(self.output_ids)

    def is_finished(self, stop_ids: List[int]) -> bool:
        if self.max_tokens is not None and self.output_tokens >= self.max_tokens:
            return True
        return bool(self.output_ids) and self.output_ids[-1] in stop_ids


class TaskManager:
    def __init__(self, tokenizer, max_batch_size: int = 16, max_seq_len: int = 8192, max_prompt_len: int = 512):
        self.tokenizer = tokenizer
        self.max_batch_size, self.max_seq_len, self.max_prompt_len = max_batch_size, max_seq_len, max_prompt_len
        self.waiting_queue: Deque[Task] = deque()
        self.active_tasks: List[Task] = []
        self._task_event = threading.Event()
        self._lock = threading.Lock()
        self._total_tasks = 0
        self._total_tokens = 0
        self._cancelled: Dict[str, None] = {}   # ids cancelled while their task was between the queue and the batch
        self._ttft: Deque[float] = deque(maxlen=RECENT)
        self._latency: Deque[float] = deque(maxlen=RECENT)
        self._itl: Deque[float] = deque(maxlen=RECENT)   # mean inter-token latency of each finished request
        self._hist = {"ttft_seconds": Histogram(), "itl_seconds": Histogram(), "latency_seconds": Histogram()}

    def add_task(self, prompt, max_tokens: Optional[int] = None, temperature: float = 1.0, top_p: float = 1.0,
                 top_k: int = 50, stream_callback: Optional[Callable] = None) -> str:
        """``prompt`` is text, or a list of token ids (used by load generators)."""
        task_id = f"task_{int(time.time())}_{uuid.uuid4().hex[:8]}"
        ids = list(prompt) if isinstance(prompt, (list, tuple)) else self.tokenizer.encode(prompt)
        if len(ids) > self.max_prompt_len:
            ids = ids[-self.max_prompt_len:]
        room = self.max_seq_len - len(ids)
        if room <= 0 or not ids or (max_tokens is not None and max_tokens <= 0):
            # nothing can be generated: no room left, nothing to condition on, or nothing asked for
            if stream_callback:
                stream_callback(STOP)
            return task_id
        task = Task(task_id, ids, room if max_tokens is None else min(max_tokens, room), temperature, top_p, top_k,
                    stream_callback)
        with self._lock:
            self.waiting_queue.append(task)
            self._total_tasks += 1
        self._task_event.set()
        return task_id

    def remove_task(self, task_id: str) -> List[Task]:
        with self._lock:
            removed = [t for t in self.active_tasks if t.task_id == task_id]
            self.waiting_queue = deque(t for t in self.waiting_queue if t.task_id != task_id)
            self.active_tasks = [t for t in self.active_tasks if t.task_id != task_id]
        return removed

    def cancel(self, task_id: str) -> Optional[Task]:
        """Withdraw a task from any thread and return it (``None`` if it is unknown or already done).
        A waiting task leaves the queue; a running one is only marked ``ABORTED`` - the scheduler
        thread, which owns the KV pages, collects it at its next clean-up, so no page is freed under a
        step that is still using it."""
        found: Optional[Task] = None
        with self._lock:
            for t in self.waiting_queue:
                if t.task_id == task_id:
                    found = t
                    break
            if found is not None:
                self.waiting_queue = deque(t for t in self.waiting_queue if t.task_id != task_id)
                found.status = TaskStatus.ABORTED
            else:
                for t in self.active_tasks:
                    if t.task_id == task_id:
                        if t.status == TaskStatus.RUNNING:
                            t.status = TaskStatus.ABORTED
                        found = t
                        break
            if found is None:
                # between the queue and the batch right now, or finished long ago: remember the id for a while
                self._cancelled[task_id] = None
                while len(self._cancelled) > 1024:
                    self._cancelled.pop(next(iter(self._cancelled)))
        self._task_event.set()
        return found

    def get_stats(self) -> Dict[str, Any]:
        return {"total_tasks": self._total_tasks, "total_tokens": self._total_tokens,
                "active_tasks": len(self.active_tasks), "waiting_queue": len(self.waiting_queue)}

    def latency_stats(self) -> Dict[str, Any]:
        def pct(xs, q):
            if not xs:
                return None
            ys = sorted(xs)
            return ys[min(len(ys) - 1, int(q * len(ys)))]

        with self._lock:
            return {"ttft_p50_s": pct(self._ttft, 0.5), "ttft_p99_s": pct(self._ttft, 0.99),
                    "itl_p50_s": pct(self._itl, 0.5), "itl_p99_s": pct(self._itl, 0.99),
                    "latency_p50_s": pct(self._latency, 0.5), "finished": len(self._latency)}

    def histograms(self) -> Dict[str, Dict[str, Any]]:
        """Time to first token, mean inter-token latency and total latency of every finished request
        since start, as cumulative histograms."""
        with self._lock:
            return {name: h.snapshot() for name, h in self._hist.items()}

    def remove_finished_tasks(self, stop_ids: List[int]) -> List[Task]:
        now = time.time()
        with self._lock:
            done: List[Task] = []
            for t in self.active_tasks:
                if t.status == TaskStatus.ABORTED:
                    t.finish_time = now
                    done.append(t)
                elif t.is_finished(stop_ids):
                    t.status, t.finish_time = TaskStatus.FINISHED, now
                    self._total_tokens += t.output_tokens
                    self._latency.append(now - t.arrival_time)
                    self._hist["latency_seconds"].observe(now - t.arrival_time)
                    if t.first_token_time is not None:
                        self._ttft.append(t.first_token_time - t.arrival_time)
                        self._hist["ttft_seconds"].observe(t.first_token_time - t.arrival_time)
                        if t.output_tokens > 1:
                            itl = (now - t.first_token_time) / (t.output_tokens - 1)
                            self._itl.append(itl)
                            self._hist["itl_seconds"].observe(itl)
                    done.append(t)
            self.active_tasks = [t for t in self.active_tasks
                                 if t.status not in (TaskStatus.FINISHED, TaskStatus.ABORTED)]
            return done

    def pull_candidates(self, n: int) -> List[Task]:
        with self._lock:
            return [self.waiting_queue.popleft() for _ in range(min(max(n, 0), len(self.waiting_queue)))]

    def activate(self, task: Task) -> None:
        with self._lock:
            cancelled = self._cancelled.pop(task.task_id, 0) is None
            task.status = TaskStatus.ABORTED if cancelled else TaskStatus.RUNNING
            self.active_tasks.append(task)

    def return_to_waiting(self, tasks: List[Task]) -> None:
        with self._lock:
            self.waiting_queue.extendleft(reversed(tasks))

    def has_work(self) -> bool:
        return bool(self.active_tasks or self.waiting_queue)

    def wait_for_tasks(self, timeout: float = 1.0) -> None:
        with self._lock:
            if self.waiting_queue or self.active_tasks:
                return
            self._task_event.clear()
        self._task_event.wait(timeout=timeout)

    def get_active_tasks(self) -> List[Task]:
        with self._lock:
            return list(self.active_tasks)

    def get_waiting_tasks(self) -> List[Task]:
        with self._lock:
            return list(self.waiting_queue)

    def clear_queues(self) -> None:
        with self._lock:
            self.waiting_queue.clear()
            self.active_tasks.clear()

    def wake(self) -> None:
        self._task_event.set()
