"""OpenAI ``/v1/chat/completions`` wire format (reference: ``astrai/inference/api/openai.py``).
Quirks kept for client compatibility: ``finish_reason`` is always ``"stop"``, content chunks
carry ``created: 0``, the non-streamed content keeps a matched stop sequence."""

from __future__ import annotations

import logging
import time
import uuid
from typing import Any, Dict, List, Tuple

from .protocol import GenContext, ResponseBuilder, StopInfo, sse_event

log = logging.getLogger(__name__)
UNSUPPORTED = ("n", "presence_penalty", "frequency_penalty", "logit_bias", "user")


def _usage(ctx: GenContext) -> Dict[str, int]:
    return {"prompt_tokens": ctx.prompt_tokens, "completion_tokens": ctx.completion_tokens,
            "total_tokens": ctx.prompt_tokens + ctx.completion_tokens}


class OpenAIResponseBuilder(ResponseBuilder):
    def prepare(self, request, engine) -> Tuple[str, GenContext, List[str]]:
        messages = [{"role": m.role, "content": m.content} for m in request.messages]
        prompt = engine.tokenizer.apply_chat_template(messages, tokenize=False)
        self._resp_id = f"chatcmpl-{uuid.uuid4().hex[:12]}"
        self._model = request.model
        fields = getattr(type(request), "model_fields", {})
        for name in UNSUPPORTED:
            value = getattr(request, name, None)
            default = fields[name].default if name in fields else None
            if value is not None and value != default:
                log.warning("ChatCompletionRequest param '%s'=%r is not supported and will be ignored", name, value)
        stop = request.stop
        stops = [] if stop is None else [stop] if isinstance(stop, str) else list(stop)
        return prompt, GenContext(self._resp_id, int(time.time()), self._model, 0), stops

    def _chunk(self, created: int, delta: Dict[str, Any], finish) -> Dict[str, Any]:
        return {"id": self._resp_id, "object": "chat.completion.chunk", "created": created, "model": self._model,
                "choices": [{"index": 0, "delta": delta, "finish_reason": finish}]}

    def format_stream_start(self, ctx):
        return [sse_event(self._chunk(ctx.created, {"role": "assistant"}, None))]

    def format_chunk(self, token):
        return sse_event(self._chunk(0, {"content": token}, None))

    def format_stream_end(self, ctx, stop: StopInfo):
        return [sse_event(self._chunk(ctx.created, {}, "stop")), sse_event(_usage(ctx))]

    def format_response(self, ctx, content, stop: StopInfo):
        return {"id": self._resp_id, "object": "chat.completion", "created": ctx.created, "model": self._model,
                "choices": [{"index": 0, "message": {"role": "assistant", "content": content},
                             "finish_reason": "stop"}],
                "usage": _usage(ctx)}
