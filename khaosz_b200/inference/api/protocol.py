"""Protocol-independent request handling: SSE framing, stop-sequence detection and the
``ResponseBuilder`` contract each wire format implements
(reference: ``astrai/inference/api/protocol.py:18-182``).  SSE events end with a blank line
as the specification requires (the reference ends ordinary events with a single newline).
"""

from __future__ import annotations

import json
from abc import ABC, abstractmethod
from dataclasses import dataclass
from typing import Any, AsyncGenerator, Dict, List, Optional, Tuple

from fastapi.responses import StreamingResponse


def sse_event(data: Dict[str, Any], event: Optional[str] = None) -> str:
    head = f"event: {event}\n" if event else ""
    return f"{head}data: {json.dumps(data, ensure_ascii=False)}\n\n"


def sse_done() -> str:
    return "data: [DONE]\n\n"


@dataclass
class GenContext:
    resp_id: str
    created: int
    model: str
    prompt_tokens: int
    completion_tokens: int = 0


@dataclass
class StopInfo:
    matched: Optional[str] = None  # the stop sequence that ended generation, if any
    body: str = ""                 # everything generated, stop sequence included
    yielded: str = ""              # what was already streamed to the client


class StopChecker:
    def __init__(self, sequences: List[str]):
        self._sequences = [s for s in sequences if s]

    def check(self, text: str) -> Optional[str]:
        return next((s for s in self._sequences if s in text), None)


class ResponseBuilder(ABC):
    """One concrete builder per wire protocol."""

    @abstractmethod
    def prepare(self, request, engine) -> Tuple[str, GenContext, List[str]]:
        """-> (prompt text, context, stop sequences)"""

    @abstractmethod
    def format_stream_start(self, ctx: GenContext) -> List[str]: ...

    @abstractmethod
    def format_chunk(self, token: str) -> str: ...

    @abstractmethod
    def format_stream_end(self, ctx: GenContext, stop: StopInfo) -> List[str]: ...

    @abstractmethod
    def format_response(self, ctx: GenContext, content: str, stop: StopInfo) -> Dict[str, Any]: ...


class ProtocolHandler:
    """``await ProtocolHandler(request, engine, builder).handle()`` -> dict or SSE response."""

    def __init__(self, request, engine, builder: ResponseBuilder):
        self.request, self.engine, self.builder = request, engine, builder

    async def handle(self):
        prompt, ctx, stops = self.builder.prepare(self.request, self.engine)
        ctx.prompt_tokens = len(self.engine.tokenizer.encode(prompt))
        req = self.request
        tokens = self.engine.generate_async(prompt=prompt, max_tokens=req.max_tokens, temperature=req.temperature,
                                            top_p=req.top_p, top_k=req.top_k)
        if req.stream:
            return StreamingResponse(self._stream(tokens, ctx, stops), media_type="text/event-stream",
                                     headers={"Cache-Control": "no-cache", "Connection": "keep-alive"})
        return await self._collect(tokens, ctx, stops)

    @staticmethod
    async def _consume(tokens: AsyncGenerator, checker: StopChecker, ctx: GenContext):
        """Yield (token, body, matched) until the stream ends or a stop sequence appears."""
        body = ""
        async for token in tokens:
            body += token
            matched = checker.check(body)
            if matched:
                yield token, body, matched
                return
            ctx.completion_tokens += 1
            yield token, body, None

    async def _stream(self, tokens, ctx, stops):
        for ev in self.builder.format_stream_start(ctx):
            yield ev
        info = StopInfo()
        async for token, body, matched in self._consume(tokens, StopChecker(stops), ctx):
            info.body = body
            if matched:
                info.matched = matched
                break
            info.yielded += token
            yield self.builder.format_chunk(token)
        for ev in self.builder.format_stream_end(ctx, info):
            yield ev
        yield sse_done()

    async def _collect(self, tokens, ctx, stops) -> Dict[str, Any]:
        info = StopInfo()
        async for _token, body, matched in self._consume(tokens, StopChecker(stops), ctx):
            info.body, info.matched = body, matched
        return self.builder.format_response(ctx, info.body, info)
