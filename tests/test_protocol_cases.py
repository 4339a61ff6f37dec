"""Case-by-case behaviour of the protocol layer: SSE framing, stop-sequence detection, the OpenAI and
Anthropic response builders, the protocol handler and request validation (the behaviours the
reference pins in ``tests/inference/test_protocol.py``)."""
import asyncio
import json

import pytest

from khaosz_b200 import GenerationRequest
from khaosz_b200.inference.api import (AnthropicResponseBuilder, OpenAIResponseBuilder, ProtocolHandler, StopChecker,
                                       StopInfo, sse_done, sse_event)
from khaosz_b200.inference.api.anthropic import extract_text
from khaosz_b200.inference.api.protocol import GenContext, ResponseBuilder
from khaosz_b200.inference.api.server import ChatCompletionRequest, MessagesRequest


class _Tokenizer:
    def apply_chat_template(self, messages, tokenize=False, **_):
        return "".join(f"[{m['role']}]{m['content']}" for m in messages)

    def encode(self, text, **_):
        return text.split()


class _Engine:
    def __init__(self, tokens=()):
        self.tokens, self.tokenizer, self.calls = list(tokens), _Tokenizer(), []

    def generate_async(self, prompt, **kw):
        self.calls.append((prompt, kw))

        async def gen():
            for t in self.tokens:
                yield t

        return gen()


def _payload(event: str) -> dict:
    line = next(l for l in event.splitlines() if l.startswith("data: "))
    return json.loads(line[6:])


def _chat(**kw):
    return ChatCompletionRequest(messages=[{"role": "user", "content": "hi there"}], **kw)


def _msgs(**kw):
    return MessagesRequest(messages=[{"role": "user", "content": "hi there"}], **kw)


# ---- framing and stop detection ---------------------------------------------------------------
def test_sse_event_is_one_data_line_and_a_blank_line():
    assert sse_event({"a": 1}) == 'data: {"a": 1}\n\n'
    assert sse_event({"a": "é"}) == 'data: {"a": "é"}\n\n'                       # no ascii escaping
    assert sse_event({"a": 1}, event="ping") == 'event: ping\ndata: {"a": 1}\n\n'
    assert sse_done() == "data: [DONE]\n\n"


def test_stop_checker_finds_the_first_listed_match():
    checker = StopChecker(["END", "stop"])
    assert checker.check("the END") == "END" and checker.check("full stop here") == "stop"
    assert checker.check("stop before END") == "END"                              # list order, not text order


def test_stop_checker_without_a_match_or_without_sequences():
    assert StopChecker(["END"]).check("nothing here") is None
    assert StopChecker([]).check("anything") is None
    assert StopChecker(["", ""]).check("anything") is None                        # empty strings never match


def test_stop_info_and_context_defaults():
    info = StopInfo()
    assert (info.matched, info.body, info.yielded) == (None, "", "")
    info.matched, info.body = "X", "abcX"
    assert info.matched == "X"
    ctx = GenContext("id", 5, "m", 7)
    assert ctx.completion_tokens == 0 and (ctx.resp_id, ctx.created, ctx.model, ctx.prompt_tokens) == ("id", 5, "m", 7)
    assert GenContext("id", 5, "m", 7, 3).completion_tokens == 3


def test_response_builder_is_abstract():
    with pytest.raises(TypeError):
        ResponseBuilder()


# ---- OpenAI -----------------------------------------------------------------------------------
def test_openai_prepare_renders_the_prompt_and_collects_stops():
    b = OpenAIResponseBuilder()
    prompt, ctx, stops = b.prepare(_chat(stop=["END", "###"], model="mine"), _Engine())
    assert prompt == "[user]hi there" and stops == ["END", "###"]
    assert ctx.resp_id.startswith("chatcmpl-") and ctx.model == "mine" and ctx.created > 0
    assert b.prepare(_chat(stop="END"), _Engine())[2] == ["END"]                  # a bare string is one sequence
    assert b.prepare(_chat(), _Engine())[2] == []


def test_openai_prepare_warns_about_ignored_parameters(caplog):
    with caplog.at_level("WARNING"):
        OpenAIResponseBuilder().prepare(_chat(n=3, presence_penalty=0.5, user="u"), _Engine())
    text = caplog.text
    assert "'n'" in text and "presence_penalty" in text and "'user'" in text and "frequency_penalty" not in text


def test_openai_stream_events():
    b = OpenAIResponseBuilder()
    _, ctx, _ = b.prepare(_chat(), _Engine())
    ctx.prompt_tokens, ctx.completion_tokens = 4, 2
    start = [_payload(e) for e in b.format_stream_start(ctx)]
    assert len(start) == 1 and start[0]["object"] == "chat.completion.chunk"
    assert start[0]["choices"][0] == {"index": 0, "delta": {"role": "assistant"}, "finish_reason": None}
    chunk = _payload(b.format_chunk("tok"))
    assert chunk["choices"][0]["delta"] == {"content": "tok"} and chunk["created"] == 0 and chunk["id"] == ctx.resp_id
    end = [_payload(e) for e in b.format_stream_end(ctx, StopInfo())]
    assert end[0]["choices"][0] == {"index": 0, "delta": {}, "finish_reason": "stop"}
    assert end[1] == {"prompt_tokens": 4, "completion_tokens": 2, "total_tokens": 6}


def test_openai_response_keeps_the_stop_sequence():
    b = OpenAIResponseBuilder()
    _, ctx, _ = b.prepare(_chat(), _Engine())
    ctx.prompt_tokens, ctx.completion_tokens = 3, 5
    out = b.format_response(ctx, "hello END", StopInfo(matched="END", body="hello END"))
    assert out["object"] == "chat.completion" and out["created"] == ctx.created
    assert out["choices"] == [{"index": 0, "message": {"role": "assistant", "content": "hello END"}, "finish_reason": "stop"}]
    assert out["usage"] == {"prompt_tokens": 3, "completion_tokens": 5, "total_tokens": 8}


# ---- Anthropic --------------------------------------------------------------------------------
def test_anthropic_prepare_puts_the_system_prompt_first():
    prompt, ctx, stops = AnthropicResponseBuilder().prepare(_msgs(system="be brief", stop_sequences=["END"]), _Engine())
    assert prompt == "[system]be brief[user]hi there" and stops == ["END"] and ctx.resp_id.startswith("msg_")
    assert AnthropicResponseBuilder().prepare(_msgs(), _Engine())[2] == []


def test_anthropic_prepare_reads_text_blocks():
    req = MessagesRequest(messages=[{"role": "user", "content": [{"type": "image", "source": {}}, {"type": "text", "text": "look"}]},
                                    {"role": "assistant", "content": []}])
    prompt, _, _ = AnthropicResponseBuilder().prepare(req, _Engine())
    assert prompt == "[user]look"                                                 # block without text is dropped
    assert extract_text("plain") == "plain" and extract_text([{"type": "tool_use"}]) == "" and extract_text(None) == ""


def test_anthropic_stream_start_and_chunk():
    b = AnthropicResponseBuilder()
    ctx = GenContext("msg_1", 0, "m", 9)
    start = b.format_stream_start(ctx)
    assert [e.split("\n")[0] for e in start] == ["event: message_start", "event: content_block_start"]
    message = _payload(start[0])["message"]
    assert message["id"] == "msg_1" and message["role"] == "assistant" and message["usage"] == {"input_tokens": 9}
    assert _payload(start[1])["content_block"] == {"type": "text", "text": ""}
    chunk = b.format_chunk("tok")
    assert chunk.startswith("event: content_block_delta\n")
    assert _payload(chunk)["delta"] == {"type": "text_delta", "text": "tok"}


def test_anthropic_stream_end_without_a_stop_sequence():
    ctx = GenContext("msg_1", 0, "m", 9, 4)
    events = AnthropicResponseBuilder().format_stream_end(ctx, StopInfo(body="abcd", yielded="abcd"))
    assert [e.split("\n")[0] for e in events] == ["event: content_block_stop", "event: message_delta", "event: message_stop"]
    delta = _payload(events[1])
    assert delta["delta"] == {"stop_reason": "end_turn", "stop_sequence": None} and delta["usage"] == {"output_tokens": 4}


def test_anthropic_stream_end_flushes_text_held_back_before_the_stop_sequence():
    ctx = GenContext("msg_1", 0, "m", 9, 4)
    events = AnthropicResponseBuilder().format_stream_end(ctx, StopInfo(matched="END", body="abc END", yielded="ab"))
    assert _payload(events[0])["delta"]["text"] == "c "                           # generated, not yet sent, before END
    assert _payload(events[2])["delta"] == {"stop_reason": "stop_sequence", "stop_sequence": "END"}
    assert len(events) == 4


def test_anthropic_stream_end_sends_nothing_extra_when_all_was_streamed():
    ctx = GenContext("msg_1", 0, "m", 9, 4)
    events = AnthropicResponseBuilder().format_stream_end(ctx, StopInfo(matched="END", body="abcEND", yielded="abc"))
    assert len(events) == 3 and events[0].startswith("event: content_block_stop")


def test_anthropic_response_trims_the_stop_sequence():
    ctx = GenContext("msg_1", 0, "m", 9, 4)
    b = AnthropicResponseBuilder()
    out = b.format_response(ctx, "hello END", StopInfo(matched="END", body="hello END"))
    assert out["content"] == [{"type": "text", "text": "hello "}]
    assert out["stop_reason"] == "stop_sequence" and out["stop_sequence"] == "END"
    assert out["usage"] == {"input_tokens": 9, "output_tokens": 4} and out["type"] == "message"
    plain = b.format_response(ctx, "hello", StopInfo(body="hello"))
    assert plain["content"][0]["text"] == "hello" and plain["stop_reason"] == "end_turn" and plain["stop_sequence"] is None


# ---- handler ----------------------------------------------------------------------------------
def test_handler_collects_until_the_stop_sequence_and_counts_tokens():
    engine = _Engine(["Hello", " wor", "ld", " END", " tail"])
    out = asyncio.run(ProtocolHandler(_chat(stop="END", max_tokens=9, temperature=0.5, top_p=0.8, top_k=3), engine,
                                      OpenAIResponseBuilder()).handle())
    assert out["choices"][0]["message"]["content"] == "Hello world END"            # generation stopped before " tail"
    assert out["usage"]["prompt_tokens"] == 2 and out["usage"]["completion_tokens"] == 3
    prompt, kw = engine.calls[0]
    assert prompt == "[user]hi there" and kw == {"max_tokens": 9, "temperature": 0.5, "top_p": 0.8, "top_k": 3}


def test_handler_without_stop_returns_everything():
    out = asyncio.run(ProtocolHandler(_msgs(), _Engine(["a", "b", "c"]), AnthropicResponseBuilder()).handle())
    assert out["content"][0]["text"] == "abc" and out["usage"]["output_tokens"] == 3 and out["stop_reason"] == "end_turn"


def test_handler_streams_chunks_then_the_end_events_then_done():
    async def run():
        resp = await ProtocolHandler(_chat(stream=True, stop="END"), _Engine(["Hel", "lo", " END", "x"]),
                                     OpenAIResponseBuilder()).handle()
        return [part async for part in resp.body_iterator]

    parts = asyncio.run(run())
    assert parts[-1] == "data: [DONE]\n\n"
    deltas = [_payload(p)["choices"][0]["delta"] for p in parts[:-2] if "choices" in _payload(p)]
    assert deltas == [{"role": "assistant"}, {"content": "Hel"}, {"content": "lo"}, {}]   # the stop token is not sent
    assert _payload(parts[-2])["completion_tokens"] == 2


# ---- request validation -----------------------------------------------------------------------
def test_generation_request_accepts_the_documented_ranges():
    r = GenerationRequest([{"role": "user", "content": "x"}], top_k=0, top_p=0.0, temperature=0.01, max_tokens=5, stream=True)
    assert (r.top_k, r.top_p, r.temperature, r.max_tokens, r.stream) == (0, 0.0, 0.01, 5, True)
    GenerationRequest([], top_k=1000, top_p=1.0, temperature=2.5)


@pytest.mark.parametrize("kw,word", [({"top_p": 1.5}, "top_p"), ({"top_p": -0.1}, "top_p"), ({"top_k": -1}, "top_k"),
                                     ({"top_k": 1.5}, "top_k"), ({"temperature": 0.0}, "temperature"),
                                     ({"temperature": -1.0}, "temperature")])
def test_generation_request_rejects_bad_sampling_parameters(kw, word):
    with pytest.raises(ValueError, match=word):
        GenerationRequest([{"role": "user", "content": "x"}], **kw)


def test_http_schemas_have_the_documented_defaults_and_bounds():
    chat = _chat()
    assert (chat.model, chat.temperature, chat.top_p, chat.top_k, chat.max_tokens, chat.stream, chat.stop) == \
        ("astrai", 1.0, 1.0, 50, 2048, False, None)
    msg = _msgs()
    assert (msg.max_tokens, msg.temperature, msg.top_k, msg.stream, msg.system, msg.stop_sequences) == \
        (1024, 1.0, 50, False, None, None)
    from pydantic import ValidationError

    for bad in ({"temperature": 2.5}, {"top_p": 1.5}, {"top_k": 0}, {"max_tokens": 0}):
        with pytest.raises(ValidationError):
            _chat(**bad)
