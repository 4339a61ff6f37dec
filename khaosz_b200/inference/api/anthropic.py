"""Anthropic ``/v1/messages`` wire format (reference: ``astrai/inference/api/anthropic.py``):
``message_start``, ``content_block_start``, ``content_block_delta`` ..., ``content_block_stop``,
``message_delta``, ``message_stop``; a matched stop sequence is trimmed from the text, and text
generated before it that was not yet streamed is flushed as a final delta."""

from __future__ import annotations

import time
import uuid
from typing import Any, Dict, List, Tuple, Union

from .protocol import GenContext, ResponseBuilder, StopInfo, sse_event


def extract_text(content: Union[str, List[Dict[str, Any]]]) -> str:
    if isinstance(content, str):
        return content
    if isinstance(content, list):
        for block in content:
            if isinstance(block, dict) and block.get("type") == "text":
                return block.get("text", "")
    return ""


def _delta(text: str) -> str:
    return sse_event({"type": "content_block_delta", "index": 0, "delta": {"type": "text_delta", "text": text}},
                     event="content_block_delta")


def _stop_fields(stop: StopInfo) -> Dict[str, Any]:
    return {"stop_reason": "stop_sequence" if stop.matched else "end_turn", "stop_sequence": stop.matched}


class AnthropicResponseBuilder(ResponseBuilder):
    def prepare(self, request, engine) -> Tuple[str, GenContext, List[str]]:
        messages: List[Dict[str, str]] = []
        if getattr(request, "system", None):
            messages.append({"role": "system", "content": request.system})
        for m in request.messages:
            text = extract_text(m.content)
            if text:
                messages.append({"role": m.role, "content": text})
        prompt = engine.tokenizer.apply_chat_template(messages, tokenize=False)
        ctx = GenContext(f"msg_{uuid.uuid4().hex[:24]}", int(time.time()), request.model, 0)
        return prompt, ctx, list(getattr(request, "stop_sequences", None) or [])

    def format_stream_start(self, ctx):
        message = {"id": ctx.resp_id, "type": "message", "role": "assistant", "model": ctx.model, "content": [],
                   "usage": {"input_tokens": ctx.prompt_tokens}}
        return [sse_event({"type": "message_start", "message": message}, event="message_start"),
                sse_event({"type": "content_block_start", "index": 0, "content_block": {"type": "text", "text": ""}},
                          event="content_block_start")]

    def format_chunk(self, token):
        return _delta(token)

    def format_stream_end(self, ctx, stop: StopInfo):
        events: List[str] = []
        if stop.matched:
            pending = stop.body[: stop.body.rfind(stop.matched)][len(stop.yielded):]
            if pending:
                events.append(_delta(pending))
        events.append(sse_event({"type": "content_block_stop", "index": 0}, event="content_block_stop"))
        events.append(sse_event({"type": "message_delta", "delta": _stop_fields(stop),
                                 "usage": {"output_tokens": ctx.completion_tokens}}, event="message_delta"))
        events.append(sse_event({"type": "message_stop"}, event="message_stop"))
        return events

    def format_response(self, ctx, content, stop: StopInfo):
        if stop.matched:
            content = content[: content.rfind(stop.matched)]
        return {"id": ctx.resp_id, "type": "message", "role": "assistant", "model": ctx.model,
                "content": [{"type": "text", "text": content}], **_stop_fields(stop),
                "usage": {"input_tokens": ctx.prompt_tokens, "output_tokens": ctx.completion_tokens}}
