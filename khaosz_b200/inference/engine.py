"""``InferenceEngine``: the user-facing facade over the scheduler thread
(reference: ``astrai/inference/engine.py:16-288``).

``generate`` returns a string, a list of strings, or — with ``stream=True`` — a generator of
tokens (``(index, token)`` pairs for batched prompts); ``generate_async`` yields tokens on an
asyncio loop without a thread-pool hop per token.
"""

from __future__ import annotations

import asyncio
import threading
from typing import Any, AsyncGenerator, Dict, Generator, List, Optional, Tuple, Union

import torch.nn as nn

from .core.scheduler import InferenceScheduler
from .core.task import STOP


class GenerateResult:
    """Thread-safe accumulator filled by stream callbacks: per-prompt text, a queue of
    ``(index, token)`` events and completion tracking (a repeated STOP is counted once)."""

    def __init__(self, count: int = 1):
        self._cond = threading.Condition()
        self._event = threading.Event()
        self.tokens: List[Tuple[int, Any]] = []
        self.results: List[str] = [""] * count
        self._done = [False] * count
        self._completed, self._total = 0, count

    def append(self, token, idx: int = 0) -> None:
        with self._cond:
            self.tokens.append((idx, token))
            if token is STOP:
                if not self._done[idx]:
                    self._done[idx] = True
                    self._completed += 1
                    self._cond.notify_all()
            else:
                self.results[idx] += token
            self._event.set()

    def pop_all(self) -> List[Tuple[int, Any]]:
        with self._cond:
            items, self.tokens = self.tokens, []
            if not items:
                self._event.clear()
            return items

    def wait(self, timeout: Optional[float] = None) -> bool:
        return self._event.wait(timeout=timeout)

    def wait_completion(self, timeout: float = 300.0) -> None:
        with self._cond:
            if not self._cond.wait_for(lambda: self._completed >= self._total, timeout=timeout):
                raise TimeoutError(f"Generation timeout after {timeout}s ({self._completed}/{self._total} completed)")

    def get_results(self) -> List[str]:
        with self._cond:
            return list(self.results)


class GenerationRequest:
    def __init__(self, messages: List[Dict[str, str]], top_k: int = 50, top_p: float = 1.0, temperature: float = 1.0,
                 max_tokens: Optional[int] = None, stream: bool = False):
        if not isinstance(top_k, int) or isinstance(top_k, bool) or top_k < 0:
            raise ValueError("top_k must be a non-negative integer")
        if not 0.0 <= top_p <= 1.0:
            raise ValueError("top_p must be a float between 0.0 and 1.0")
        if not isinstance(temperature, (int, float)) or temperature <= 0:
            raise ValueError("temperature must be a positive number")
        self.messages, self.top_k, self.top_p = messages, top_k, top_p
        self.temperature, self.max_tokens, self.stream = temperature, max_tokens, stream


class InferenceEngine:
    def __init__(self, model: nn.Module, tokenizer, max_batch_size: int = 1, max_seq_len: Optional[int] = None,
                 max_prompt_len: int = 2048, page_size: int = 128):
        self.model, self.tokenizer = model, tokenizer
        self.scheduler = InferenceScheduler(model=model, tokenizer=tokenizer, max_batch_size=max_batch_size,
                                            max_seq_len=max_seq_len, max_prompt_len=max_prompt_len,
                                            page_size=page_size)
        self.scheduler.start()

    def __enter__(self):
        return self

    def __exit__(self, exc_type, exc, tb):
        self.shutdown()
        return False

    # -- submission -----------------------------------------------------------------------------
    def _submit_tasks(self, prompts: List, max_tokens, temperature, top_p, top_k) -> Tuple[GenerateResult, List[str]]:
        result = GenerateResult(count=len(prompts))
        ids = [self.scheduler.add_task(prompt=p, max_tokens=max_tokens, temperature=temperature, top_p=top_p,
                                       top_k=top_k, stream_callback=self._make_callback(result, i))
               for i, p in enumerate(prompts)]
        return result, ids

    @staticmethod
    def _make_callback(result: GenerateResult, idx: int):
        return lambda token: result.append(token, idx)

    def _release(self, task_ids: List[str]) -> None:
        for tid in task_ids:
            self.scheduler.remove_task(tid)

    # -- public API -----------------------------------------------------------------------------
    def generate(self, prompt: Union[str, List[str]], stream: bool = False, max_tokens: Optional[int] = None,
                 temperature: float = 1.0, top_p: float = 1.0, top_k: int = 50):
        batch = isinstance(prompt, list)
        prompts = prompt if batch else [prompt]
        if stream:
            return self._generate_streaming(prompts, batch, max_tokens, temperature, top_p, top_k)
        return self._generate_non_streaming(prompts, batch, max_tokens, temperature, top_p, top_k)

    def _generate_streaming(self, prompts, is_batch, max_tokens, temperature, top_p, top_k) -> Generator:
        result, task_ids = self._submit_tasks(prompts, max_tokens, temperature, top_p, top_k)

        def events():
            open_streams = set(range(len(prompts)))
            try:
                while open_streams:
                    for idx, token in result.pop_all():
                        if token is STOP:
                            open_streams.discard(idx)
                        else:
                            yield (idx, token) if is_batch else token
                    if open_streams:
                        result.wait(timeout=0.05)
            finally:
                self._release(task_ids)

        return events()

    def _generate_non_streaming(self, prompts, is_batch, max_tokens, temperature, top_p, top_k):
        result, task_ids = self._submit_tasks(prompts, max_tokens, temperature, top_p, top_k)
        try:
            result.wait_completion()
        finally:
            self._release(task_ids)
        texts = result.get_results()
        return texts if is_batch else texts[0]

    def generate_async(self, prompt: str, max_tokens: Optional[int] = None, temperature: float = 1.0,
                       top_p: float = 1.0, top_k: int = 50) -> AsyncGenerator[str, None]:
        """Async token stream: the scheduler thread posts tokens straight onto the event loop."""

        async def agen():
            loop = asyncio.get_running_loop()
            queue: asyncio.Queue = asyncio.Queue()
            task_id = self.scheduler.add_task(
                prompt=prompt, max_tokens=max_tokens, temperature=temperature, top_p=top_p, top_k=top_k,
                stream_callback=lambda tok: loop.call_soon_threadsafe(queue.put_nowait, tok))
            try:
                while True:
                    token = await queue.get()
                    if token is STOP:
                        break
                    yield token
            finally:
                self.scheduler.remove_task(task_id)

        return agen()

    def generate_with_request(self, request: GenerationRequest):
        prompt = self.tokenizer.apply_chat_template(request.messages, tokenize=False)
        return self.generate(prompt=prompt, stream=request.stream, max_tokens=request.max_tokens,
                             temperature=request.temperature, top_p=request.top_p, top_k=request.top_k)

    def get_stats(self) -> Dict[str, Any]:
        return self.scheduler.get_stats()

    def get_histograms(self) -> Dict[str, Dict[str, Any]]:
        """Latency histograms of the finished requests (``/metrics`` renders them)."""
        return self.scheduler.get_histograms()

    def shutdown(self) -> None:
        self.scheduler.stop()
