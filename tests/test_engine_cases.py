"""Case-by-case behaviour of ``GenerateResult``, ``InferenceEngine.generate`` and the scheduler under
concurrent use (the behaviours the reference pins in ``tests/inference/test_engine.py`` and
``tests/inference/test_scheduler.py``)."""
import asyncio
import threading
import time

import pytest
import torch

from conftest import tiny_config
from khaosz_b200 import AutoRegressiveLM, GenerationRequest, InferenceEngine
from khaosz_b200.inference import STOP, GenerateResult


# ---- GenerateResult ---------------------------------------------------------------------------
def test_result_collects_the_text_of_one_prompt():
    r = GenerateResult()
    r.append("Hel")
    r.append("lo")
    assert r.get_results() == ["Hello"] and r.tokens == [(0, "Hel"), (0, "lo")]


def test_result_keeps_prompts_apart():
    r = GenerateResult(count=3)
    for idx, tok in ((0, "a"), (2, "c"), (1, "b"), (0, "A"), (2, "C")):
        r.append(tok, idx)
    assert r.get_results() == ["aA", "b", "cC"]


def test_result_stop_completes_a_prompt_without_adding_text():
    r = GenerateResult(count=2)
    r.append("x", 0)
    r.append(STOP, 0)
    assert r._completed == 1 and r.get_results() == ["x", ""]
    r.append(STOP, 1)
    assert r._completed == 2
    r.wait_completion(timeout=0.1)                      # returns at once


def test_result_counts_a_repeated_stop_once():
    r = GenerateResult(count=2)
    r.append(STOP, 0)
    r.append(STOP, 0)
    r.append(STOP, 0)
    assert r._completed == 1
    with pytest.raises(TimeoutError):
        r.wait_completion(timeout=0.05)


def test_result_pop_all_hands_over_the_events_and_clears_them():
    r = GenerateResult(count=2)
    r.append("a", 0)
    r.append("b", 1)
    r.append(STOP, 1)
    assert r.pop_all() == [(0, "a"), (1, "b"), (1, STOP)]
    assert r.pop_all() == [] and r.get_results() == ["a", "b"]      # the text stays


def test_result_wait_blocks_until_something_arrives():
    r = GenerateResult()
    assert r.wait(timeout=0.05) is False
    threading.Timer(0.05, lambda: r.append("late")).start()
    start = time.time()
    assert r.wait(timeout=5.0) is True and time.time() - start < 2.0
    r.pop_all()
    r.pop_all()                                         # empty pop re-arms the wait
    assert r.wait(timeout=0.02) is False


def test_result_wait_completion_waits_for_every_prompt():
    r = GenerateResult(count=2)
    r.append(STOP, 0)
    threading.Timer(0.05, lambda: r.append(STOP, 1)).start()
    r.wait_completion(timeout=5.0)
    assert r._completed == 2
    with pytest.raises(TimeoutError, match="0/1"):
        GenerateResult(1).wait_completion(timeout=0.02)


def test_result_is_safe_under_concurrent_appends():
    r = GenerateResult(count=8)

    def feed(idx):
        for _ in range(200):
            r.append("x", idx)
        r.append(STOP, idx)

    threads = [threading.Thread(target=feed, args=(i,)) for i in range(8)]
    for t in threads:
        t.start()
    r.wait_completion(timeout=10.0)
    for t in threads:
        t.join()
    assert all(len(text) == 200 for text in r.get_results()) and len(r.tokens) == 8 * 201


# ---- engine -----------------------------------------------------------------------------------
@pytest.fixture
def engine(tokenizer):
    torch.manual_seed(0)
    model = AutoRegressiveLM(tiny_config(vocab_size=len(tokenizer))).eval()
    with InferenceEngine(model, tokenizer, max_batch_size=4, max_seq_len=64, page_size=4) as eng:
        yield eng


def _greedy(model, tokenizer, prompt, n):
    ids = torch.tensor([tokenizer.encode(prompt)])
    out = []
    with torch.no_grad():
        for _ in range(n):
            nxt = int(model(ids)["logits"][0, -1].argmax())
            out.append(nxt)
            if nxt in tokenizer.stop_ids:
                break
            ids = torch.cat([ids, torch.tensor([[nxt]])], dim=1)
    return "".join(tokenizer.decode([t]) for t in out)


def test_generate_one_prompt_returns_a_string(engine, tokenizer):
    out = engine.generate("hello world", max_tokens=6, top_k=1)
    assert isinstance(out, str) and out == _greedy(engine.model, tokenizer, "hello world", 6)


def test_generate_a_list_returns_a_list_in_order(engine, tokenizer):
    prompts = ["the quick brown fox", "hello", "this is a test"]
    out = engine.generate(prompts, max_tokens=5, top_k=1)
    assert isinstance(out, list) and out == [_greedy(engine.model, tokenizer, p, 5) for p in prompts]
    assert engine.generate(["hello"], max_tokens=5, top_k=1) == [out[1]]          # a list of one stays a list


def test_generate_stream_yields_the_pieces_of_the_same_text(engine):
    whole = engine.generate("hello world", max_tokens=6, top_k=1)
    pieces = list(engine.generate("hello world", stream=True, max_tokens=6, top_k=1))
    assert all(isinstance(p, str) for p in pieces) and "".join(pieces) == whole and len(pieces) <= 6


def test_generate_stream_of_a_batch_tags_pieces_with_their_prompt(engine):
    prompts = ["hello world", "the lazy dog"]
    whole = engine.generate(prompts, max_tokens=4, top_k=1)
    texts = ["", ""]
    for idx, piece in engine.generate(prompts, stream=True, max_tokens=4, top_k=1):
        texts[idx] += piece
    assert texts == whole


def test_generate_async_streams_from_an_event_loop(engine):
    whole = engine.generate("hello world", max_tokens=5, top_k=1)

    async def collect():
        return [t async for t in engine.generate_async("hello world", max_tokens=5, top_k=1)]

    assert "".join(asyncio.run(collect())) == whole


def test_generate_with_request_renders_the_chat_template(engine, tokenizer):
    req = GenerationRequest([{"role": "user", "content": "hello"}], top_k=1, max_tokens=4)
    prompt = tokenizer.apply_chat_template(req.messages, tokenize=False)
    assert engine.generate_with_request(req) == engine.generate(prompt, max_tokens=4, top_k=1)
    streamed = engine.generate_with_request(GenerationRequest(req.messages, top_k=1, max_tokens=4, stream=True))
    assert "".join(streamed) == engine.generate(prompt, max_tokens=4, top_k=1)


def test_max_tokens_bounds_the_output(engine, tokenizer):
    engine.generate("hello world", max_tokens=1, top_k=1)
    assert engine.get_stats()["total_tokens"] == 1
    engine.generate("hello world", max_tokens=3, top_k=1)
    assert engine.get_stats()["total_tokens"] <= 1 + 3


def test_a_repeated_prompt_is_served_from_the_prefix_cache_with_the_same_result(engine, tokenizer):
    prompt = "the quick brown fox jumps over the lazy dog"          # several full pages of four tokens
    first = engine.generate(prompt, max_tokens=6, top_k=1)
    time.sleep(0.05)
    cache = engine.scheduler._page_cache
    assert cache._pool.lookup(tokenizer.encode(prompt))               # its full pages are findable
    second = engine.generate(prompt, max_tokens=6, top_k=1)
    longer = engine.generate(prompt + " hello world", max_tokens=6, top_k=1)
    assert second == first == _greedy(engine.model, tokenizer, prompt, 6)
    assert longer == _greedy(engine.model, tokenizer, prompt + " hello world", 6)


def test_sampling_parameters_are_per_request(engine):
    greedy = engine.generate(["hello world"] * 2, max_tokens=8, top_k=1)
    assert greedy[0] == greedy[1]
    torch.manual_seed(1)
    hot = {engine.generate("hello world", max_tokens=8, temperature=5.0, top_k=0) for _ in range(6)}
    assert len(hot) > 1                                               # high temperature: the runs differ


# ---- scheduler under concurrent use -------------------------------------------------------------
def test_concurrent_add_task_loses_nothing(engine):
    sched = engine.scheduler
    done, lock = [], threading.Lock()

    def submit(i):
        finished = threading.Event()

        def cb(token):
            if token is STOP:
                finished.set()

        sched.add_task(f"hello {i}", max_tokens=3, top_k=1, stream_callback=cb)
        assert finished.wait(timeout=60)
        with lock:
            done.append(i)

    threads = [threading.Thread(target=submit, args=(i,)) for i in range(12)]
    for t in threads:
        t.start()
    for t in threads:
        t.join(timeout=90)
    assert sorted(done) == list(range(12)) and sched.get_stats()["total_tasks"] == 12


def test_concurrent_add_and_remove(engine):
    sched = engine.scheduler
    errors = []

    def churn(i):
        try:
            for _ in range(5):
                tid = sched.add_task(f"the quick brown fox {i}", max_tokens=20, top_k=1)
                time.sleep(0.002 * (i % 3))
                sched.remove_task(tid)
        except Exception as exc:  # pragma: no cover
            errors.append(exc)

    threads = [threading.Thread(target=churn, args=(i,)) for i in range(6)]
    for t in threads:
        t.start()
    for t in threads:
        t.join(timeout=60)
    assert not errors
    deadline = time.time() + 10
    while sched.get_stats()["active_tasks"] + sched.get_stats()["waiting_queue"] and time.time() < deadline:
        time.sleep(0.05)
    stats = sched.get_stats()
    assert stats["active_tasks"] == 0 and stats["waiting_queue"] == 0
    assert engine.generate("hello", max_tokens=2, top_k=1) is not None     # the loop is still alive


def test_concurrent_stats_reads_while_generating(engine):
    stop = threading.Event()
    seen, errors = [], []

    def poll():
        while not stop.is_set():
            try:
                seen.append(engine.get_stats())
            except Exception as exc:  # pragma: no cover
                errors.append(exc)

    pollers = [threading.Thread(target=poll) for _ in range(3)]
    for t in pollers:
        t.start()
    engine.generate(["hello world"] * 4, max_tokens=6, top_k=1)
    stop.set()
    for t in pollers:
        t.join(timeout=10)
    assert not errors and seen
    assert all({"total_tasks", "total_tokens", "active_tasks", "waiting_queue"} <= set(s) for s in seen)
    assert all(0 <= s["active_tasks"] <= 4 for s in seen)


def test_shutdown_stops_the_loop_and_is_repeatable(tokenizer):
    model = AutoRegressiveLM(tiny_config(vocab_size=len(tokenizer))).eval()
    eng = InferenceEngine(model, tokenizer, max_batch_size=2, max_seq_len=32, page_size=4)
    thread = eng.scheduler._loop_thread
    assert thread.is_alive()
    eng.shutdown()
    thread.join(timeout=10)
    assert not thread.is_alive()
    eng.shutdown()


def test_requests_after_a_crashed_loop_are_closed_at_once(tokenizer):
    class Broken(AutoRegressiveLM):
        def forward(self, *a, **k):
            raise RuntimeError("boom")

    eng = InferenceEngine(Broken(tiny_config(vocab_size=len(tokenizer))), tokenizer, max_batch_size=2, max_seq_len=32,
                          page_size=4)
    assert eng.generate("hello", max_tokens=4) == ""                  # the crash closes the first request
    start = time.time()
    assert eng.generate("hello again", max_tokens=4) == ""            # later ones do not wait for a dead loop
    assert eng.generate(["a", "b"], max_tokens=4) == ["", ""] and time.time() - start < 5
    eng.shutdown()


def test_cancelling_a_running_request_closes_its_stream_and_frees_its_pages(engine):
    sched = engine.scheduler
    events, started = [], threading.Event()

    def cb(token):
        events.append(token)
        started.set()

    tid = sched.add_task("the quick brown fox", max_tokens=50, top_k=1, stream_callback=cb)
    assert started.wait(timeout=30)
    sched.remove_task(tid)
    assert events[-1] is STOP
    deadline = time.time() + 10
    while sched.get_stats()["active_tasks"] and time.time() < deadline:
        time.sleep(0.02)
    time.sleep(0.05)
    cache = sched._page_cache
    assert sched.get_stats()["active_tasks"] == 0 and cache.free_pages() == cache._storage.n_pages
    sched.remove_task(tid)                                            # cancelling again is harmless
    sched.remove_task("task_never_existed")


def test_closing_a_stream_early_cancels_the_request(engine):
    gen = engine.generate("the quick brown fox", stream=True, max_tokens=50, top_k=1)
    first = next(gen)
    assert isinstance(first, str)
    gen.close()                                         # the consumer walks away
    deadline = time.time() + 10
    while engine.get_stats()["active_tasks"] and time.time() < deadline:
        time.sleep(0.02)
    time.sleep(0.05)
    cache = engine.scheduler._page_cache
    assert engine.get_stats()["active_tasks"] == 0 and cache.free_pages() == cache._storage.n_pages
    assert engine.get_stats()["total_tokens"] < 50      # it did not run to the end


def test_an_abandoned_async_stream_does_not_hurt_the_engine(engine):
    async def take_one():
        agen = engine.generate_async("the quick brown fox", max_tokens=50, top_k=1)
        token = await agen.__anext__()
        await agen.aclose()
        return token

    for _ in range(3):                                  # each run closes its event loop behind it
        assert isinstance(asyncio.run(take_one()), str)
    assert engine.scheduler._fatal_error is None
    assert isinstance(engine.generate("hello", max_tokens=3, top_k=1), str)


def test_a_failing_stream_callback_only_costs_its_own_request(engine):
    def bad(token):
        raise RuntimeError("consumer went away")

    engine.scheduler.add_task("hello world", max_tokens=5, top_k=1, stream_callback=bad)
    out = engine.generate("the lazy dog", max_tokens=4, top_k=1)
    assert isinstance(out, str) and out and engine.scheduler._fatal_error is None
    deadline = time.time() + 10
    while engine.get_stats()["active_tasks"] and time.time() < deadline:
        time.sleep(0.02)
    assert engine.get_stats()["active_tasks"] == 0


def test_requests_with_nothing_to_do_return_at_once_and_do_not_hurt_the_loop(engine):
    assert engine.generate([], max_tokens=3) == []
    assert engine.generate("", max_tokens=3, top_k=1) == ""              # an empty prompt: nothing to condition on
    assert engine.generate("hello", max_tokens=0, top_k=1) == ""
    assert engine.generate(["", "hello world"], max_tokens=3, top_k=1)[0] == ""
    assert engine.scheduler._fatal_error is None
    assert engine.generate("hello world", max_tokens=3, top_k=1) != ""


def test_requests_after_shutdown_are_closed_at_once(tokenizer):
    model = AutoRegressiveLM(tiny_config(vocab_size=len(tokenizer))).eval()
    eng = InferenceEngine(model, tokenizer, max_batch_size=2, max_seq_len=32, page_size=4)
    assert eng.generate("hello world", max_tokens=3, top_k=1) != ""
    eng.shutdown()
    start = time.time()
    assert eng.generate("hello world", max_tokens=3, top_k=1) == "" and time.time() - start < 5
