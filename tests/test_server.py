import json

import pytest
from fastapi.testclient import TestClient

from khaosz_b200.inference.api import (AnthropicResponseBuilder, OpenAIResponseBuilder, StopChecker, StopInfo, app,
                                       sse_done, sse_event)
from khaosz_b200.inference.api.protocol import GenContext


class FakeTokenizer:
    def apply_chat_template(self, messages, tokenize=False, **_):
        return "".join(f"[{m['role']}]{m['content']}" for m in messages)

    def encode(self, text, **_):
        return list(range(len(text.split()) + 1))


class FakeEngine:
    def __init__(self, tokens):
        self.tokens, self.tokenizer, self.calls = tokens, FakeTokenizer(), []

    def generate_async(self, prompt, **kw):
        self.calls.append((prompt, kw))

        async def gen():
            for t in self.tokens:
                yield t

        return gen()

    def get_stats(self):
        return {"total_tasks": 1, "total_tokens": 3, "active_tasks": 0, "waiting_queue": 0}

    def shutdown(self):
        pass


@pytest.fixture
def client():
    app.state.server_config = {"_test": True}
    app.state.engine = FakeEngine(["Hello", " wor", "ld", "!", " END", " tail"])
    with TestClient(app) as c:
        yield c
    app.state.engine = None


def _events(text):
    out = []
    for line in text.splitlines():
        if line.startswith("data: ") and line != "data: [DONE]":
            out.append(json.loads(line[6:]))
    return out


def test_health_and_stats(client):
    assert client.get("/health").json() == {"status": "ok", "model_loaded": True}
    assert client.get("/stats").json()["total_tasks"] == 1
    app.state.engine = None
    assert client.get("/health").json()["model_loaded"] is False
    assert client.get("/stats").status_code == 503


def test_openai_non_stream_keeps_stop_sequence(client):
    r = client.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": "hi"}], "stop": "END",
                                                  "max_tokens": 16, "top_k": 5})
    body = r.json()
    assert body["object"] == "chat.completion" and body["choices"][0]["finish_reason"] == "stop"
    assert body["choices"][0]["message"] == {"role": "assistant", "content": "Hello world! END"}
    assert body["usage"]["completion_tokens"] == 4 and body["usage"]["total_tokens"] == body["usage"]["prompt_tokens"] + 4
    prompt, kw = app.state.engine.calls[0]
    assert prompt == "[user]hi" and kw["max_tokens"] == 16 and kw["top_k"] == 5 and kw["temperature"] == 1.0


def test_openai_stream(client):
    r = client.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": "hi"}], "stream": True,
                                                  "stop": ["END"]})
    assert r.headers["content-type"].startswith("text/event-stream") and r.text.rstrip().endswith("data: [DONE]")
    ev = _events(r.text)
    assert ev[0]["choices"][0]["delta"] == {"role": "assistant"}
    assert "".join(e["choices"][0]["delta"].get("content", "") for e in ev if "choices" in e) == "Hello world!"
    assert ev[-2]["choices"][0]["finish_reason"] == "stop" and ev[-1]["completion_tokens"] == 4


def test_anthropic_non_stream_trims_stop_sequence(client):
    r = client.post("/v1/messages", json={"messages": [{"role": "user", "content": [{"type": "text", "text": "hi"}]}],
                                          "system": "be nice", "stop_sequences": ["END"], "max_tokens": 32})
    body = r.json()
    assert body["type"] == "message" and body["content"] == [{"type": "text", "text": "Hello world! "}]
    assert body["stop_reason"] == "stop_sequence" and body["stop_sequence"] == "END"
    assert app.state.engine.calls[0][0] == "[system]be nice[user]hi"
    body = client.post("/v1/messages", json={"messages": [{"role": "user", "content": "hi"}]}).json()
    assert body["stop_reason"] == "end_turn" and body["content"][0]["text"].endswith(" tail")


def test_anthropic_stream_event_order(client):
    r = client.post("/v1/messages", json={"messages": [{"role": "user", "content": "hi"}], "stream": True,
                                          "stop_sequences": ["ld"]})
    names = [l[7:] for l in r.text.splitlines() if l.startswith("event: ")]
    assert names[:2] == ["message_start", "content_block_start"]
    assert names[-3:] == ["content_block_stop", "message_delta", "message_stop"]
    ev = _events(r.text)
    text = "".join(e["delta"]["text"] for e in ev if e.get("type") == "content_block_delta")
    assert text == "Hello wor"
    delta = [e for e in ev if e.get("type") == "message_delta"][0]
    assert delta["delta"]["stop_reason"] == "stop_sequence" and delta["usage"]["output_tokens"] == 2


def test_request_validation(client):
    assert client.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": "x"}], "top_k": 0}).status_code == 422
    assert client.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": "x"}], "temperature": 3}).status_code == 422
    assert client.post("/v1/messages", json={"messages": [], "max_tokens": 0}).status_code == 422


def test_protocol_helpers():
    assert sse_event({"a": 1}) == 'data: {"a": 1}\n\n' and sse_event({"a": 1}, event="x").startswith("event: x\ndata: ")
    assert sse_done() == "data: [DONE]\n\n"
    assert StopChecker(["", "ab"]).check("xxabyy") == "ab" and StopChecker([]).check("anything") is None
    b = AnthropicResponseBuilder()
    ctx = GenContext("id", 0, "m", 3, 2)
    events = b.format_stream_end(ctx, StopInfo(matched="END", body="abc END", yielded="ab"))
    assert '"text": "c "' in events[0]   # un-streamed text before the stop sequence is flushed
    o = OpenAIResponseBuilder()
    o._resp_id, o._model = "r", "m"
    assert json.loads(o.format_chunk("t")[6:])["created"] == 0


def test_metrics_endpoint_serves_prometheus_text(client):
    from khaosz_b200.inference.core.task import Histogram

    h = Histogram()
    for v in (0.004, 0.02, 0.02, 7.0, 1000.0):
        h.observe(v)
    snap = h.snapshot()
    assert snap["count"] == 5 and snap["cumulative"][0] == 1 and snap["cumulative"][-1] == 4   # 1000 s is above every bound
    app.state.engine.get_histograms = lambda: {"ttft_seconds": snap}
    r = client.get("/metrics")
    assert r.status_code == 200 and r.headers["content-type"].startswith("text/plain")
    lines = r.text.splitlines()
    assert "khaosz_b200_requests_total 1" in lines and "# TYPE khaosz_b200_ttft_seconds histogram" in lines
    assert 'khaosz_b200_ttft_seconds_bucket{le="0.025"} 3' in lines
    assert 'khaosz_b200_ttft_seconds_bucket{le="+Inf"} 5' in lines and "khaosz_b200_ttft_seconds_count 5" in lines
    buckets = [int(l.rsplit(" ", 1)[1]) for l in lines if l.startswith("khaosz_b200_ttft_seconds_bucket")]
    assert buckets == sorted(buckets)     # cumulative


# ---- the real engine behind the HTTP routes ----
@pytest.fixture
def live_client(tokenizer):
    import torch

    from conftest import tiny_config
    from khaosz_b200 import AutoRegressiveLM, InferenceEngine

    torch.manual_seed(0)
    model = AutoRegressiveLM(tiny_config(vocab_size=len(tokenizer))).eval()
    engine = InferenceEngine(model, tokenizer, max_batch_size=4, max_seq_len=64, page_size=4)
    app.state.server_config = {"_test": True}
    app.state.engine = engine
    with TestClient(app) as c:
        yield c, engine
    app.state.engine = None            # the app's shutdown hook has already stopped the engine


def test_http_routes_with_a_real_engine_agree_with_direct_generation(live_client, tokenizer):
    client, engine = live_client
    messages = [{"role": "user", "content": "hello world"}]
    prompt = tokenizer.apply_chat_template(messages, tokenize=False)
    want = engine.generate(prompt, max_tokens=6, top_k=1)
    body = client.post("/v1/chat/completions", json={"messages": messages, "max_tokens": 6, "top_k": 1}).json()
    assert body["choices"][0]["message"]["content"] == want
    assert body["usage"]["prompt_tokens"] == len(tokenizer.encode(prompt)) and 0 < body["usage"]["completion_tokens"] <= 6
    streamed = client.post("/v1/chat/completions", json={"messages": messages, "max_tokens": 6, "top_k": 1, "stream": True})
    text = "".join(e["choices"][0]["delta"].get("content", "") for e in _events(streamed.text) if "choices" in e)
    assert text == want
    msg = client.post("/v1/messages", json={"messages": messages, "max_tokens": 6, "top_k": 1}).json()
    assert msg["content"][0]["text"] == want and msg["usage"]["output_tokens"] == body["usage"]["completion_tokens"]
    import time

    deadline = time.time() + 5                      # the scheduler collects a finished request at its next pass
    while client.get("/stats").json()["active_tasks"] and time.time() < deadline:
        time.sleep(0.02)
    stats = client.get("/stats").json()
    assert stats["total_tasks"] == 4 and stats["active_tasks"] == 0 and stats["ttft_p50_s"] is not None
    assert stats["finished"] == 4 and stats["total_tokens"] == 4 * body["usage"]["completion_tokens"]
    assert "khaosz_b200_ttft_seconds_count 4" in client.get("/metrics").text


def test_http_requests_in_parallel_share_the_batch(live_client, tokenizer):
    import threading

    client, engine = live_client
    prompts = ["hello world", "the quick brown fox", "this is a test", "the lazy dog", "hello", "world"]
    want = {p: engine.generate(tokenizer.apply_chat_template([{"role": "user", "content": p}], tokenize=False),
                               max_tokens=5, top_k=1) for p in prompts}
    got, errors = {}, []

    def call(p):
        try:
            r = client.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": p}], "max_tokens": 5,
                                                          "top_k": 1})
            got[p] = r.json()["choices"][0]["message"]["content"]
        except Exception as exc:  # pragma: no cover
            errors.append(exc)

    threads = [threading.Thread(target=call, args=(p,)) for p in prompts]
    for t in threads:
        t.start()
    for t in threads:
        t.join(timeout=120)
    assert not errors and got == want
    cache = engine.scheduler._page_cache
    import time

    time.sleep(0.1)
    assert cache.free_pages() == cache._storage.n_pages


def test_odd_requests_get_an_answer_and_leave_the_engine_alive(live_client):
    client, engine = live_client
    ok = {"messages": [{"role": "user", "content": "hello world"}], "max_tokens": 3, "top_k": 1}
    odd = [
        {"messages": [], "max_tokens": 3},                                          # nothing to condition on
        {"messages": [{"role": "user", "content": ""}], "max_tokens": 3},
        {"messages": [{"role": "user", "content": "hello " * 400}], "max_tokens": 5},  # longer than the engine's window
        {**ok, "max_tokens": 100000},                                               # clamped to the room that is left
        {**ok, "stop": ""}, {**ok, "stop": ["", "zzz"]},                            # empty stop strings never match
        {**ok, "temperature": 0.0},                                                 # allowed by the schema: clamped
        {**ok, "top_p": 0.0},
    ]
    for body in odd:
        r = client.post("/v1/chat/completions", json=body)
        assert r.status_code == 200, (body, r.text)
        assert isinstance(r.json()["choices"][0]["message"]["content"], str)
        s = client.post("/v1/chat/completions", json={**body, "stream": True})
        assert s.status_code == 200 and s.text.rstrip().endswith("data: [DONE]")
    assert client.post("/v1/messages", json={"messages": [{"role": "user", "content": []}], "max_tokens": 3}).status_code == 200
    assert engine.scheduler._fatal_error is None
    assert client.post("/v1/chat/completions", json=ok).json()["choices"][0]["message"]["content"] != ""
