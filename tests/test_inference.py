import threading
import time

import pytest
import torch

from conftest import tiny_config
from khaosz_b200 import AutoRegressiveLM, GenerationRequest, InferenceEngine
from khaosz_b200.inference import (STOP, Allocator, GenerateResult, KVCache, PagePool, PrefixCache, SamplingPipeline,
                                   Storage, TaskManager, TaskStatus, TaskTable, TemperatureStrategy, TopKStrategy,
                                   TopPStrategy, page_hash, sample)


# ---- allocator / prefix cache / tables ----
def test_allocator_exhaustion_refs_and_lru():
    a = Allocator(3)
    pages = [a.alloc() for _ in range(3)]
    assert sorted(pages) == [0, 1, 2] and a.alloc() == -1
    a.inc_ref(pages[0])
    a.free(pages[0])
    assert a.ref_count(pages[0]) == 1 and a.alloc() == -1
    a.free(pages[0], keep_cached=True)   # parked in the LRU
    a.free(pages[1])                     # truly free
    evicted = []
    a.on_evict = evicted.append
    assert a.alloc() == pages[1] and evicted == []      # free pages first
    assert a.alloc() == pages[0] and evicted == [pages[0]]  # then the LRU victim


def test_prefix_cache_lookup_chained():
    pc = PrefixCache(4)
    toks = list(range(10))
    assert pc.lookup(toks) == []
    pc.record(7, toks, 0)
    pc.record(9, toks, 1)
    assert pc.lookup(toks) == [7, 9]                       # partial third page ignored
    assert pc.lookup(toks[:4] + [99] * 4) == [7]           # stops at the first miss
    assert pc.lookup([5] + toks[1:8]) == []                # same second page after a different first page: no alias
    assert page_hash(toks, 1, 4) != page_hash([5] + toks[1:], 1, 4)
    pc.evict(7)
    assert pc.lookup(toks) == [] and pc.has_page(9)


def test_page_pool_keeps_prefix_pages_cached():
    pool = PagePool(Allocator(2), PrefixCache(2))
    p = pool.alloc()
    pool.record(p, [1, 2], 0)
    pool.free(p)
    assert pool.lookup([1, 2]) == [p]   # survived the free
    q, r = pool.alloc(), pool.alloc()   # second alloc evicts the cached page
    assert {q, r} == {0, 1} and pool.lookup([1, 2]) == []


def test_task_table_tensor():
    t = TaskTable(4)
    t.set("a", [3, 1], 4)
    t.set("b", [2], 0)
    tt = t.table_tensor(["a", "b", "zz"], "cpu")
    assert tt.tolist() == [[3, 1], [2, -1], [-1, -1]] and t.get_cached("a") == 4
    assert t.pop("a") == ([3, 1], 4) and t.get("a") == []


def test_kvcache_accounting():
    kv = KVCache(1, 4, 4, 2, 8, "cpu", torch.float32)
    assert kv.task_alloc("t1", list(range(6)))            # 2 pages
    assert kv.task_extend("t1", 7) and len(kv._table.get("t1")) == 2
    assert kv.task_extend("t1", 8) and len(kv._table.get("t1")) == 3
    assert not kv.task_alloc("t2", list(range(9)))         # needs 3, only 1 left; nothing leaks
    assert kv.free_pages() == 1
    kv.task_record_hashes("t1", list(range(6)))
    kv.task_free("t1")
    assert kv.task_alloc("t3", list(range(6))) and kv.task_cached("t3") == 4   # first page reused


def test_storage_write_gather_roundtrip():
    st = Storage(2, 6, 4, 2, 8, "cpu", torch.float32)
    table = torch.tensor([[0, 2, 4], [1, 3, -1]])
    k, v = torch.randn(2, 6, 2, 8), torch.randn(2, 6, 2, 8)
    st.write(1, table, 0, k, v)
    gk, gv = st.gather(1, table, 6)
    assert torch.equal(gk, k) and torch.equal(gv, v)
    k2, v2 = torch.randn(2, 3, 2, 8), torch.randn(2, 3, 2, 8)
    st.write(1, table, 6, k2, v2)   # positions 6..8: page 1 tail + page 2 (missing for row 1)
    gk, _ = st.gather(1, table, 9)
    assert torch.equal(gk[0, 6:], k2[0]) and torch.equal(gk[1, 6:8], k2[1, :2]) and (gk[1, 8] == 0).all()
    assert st.gather(1, table, 5)[0].shape[1] == 5


def test_paged_forward_matches_dense_forward():
    torch.manual_seed(0)
    model = AutoRegressiveLM(tiny_config()).eval()
    ids = torch.randint(0, 300, (2, 11))
    dense = model(ids)["logits"]
    kv = KVCache(2, 16, 4, 2, 8, "cpu", torch.float32)
    for name in ("a", "b"):
        kv.task_alloc(name, list(range(12)))
    table = kv.make_table_tensor(["a", "b"], "cpu")
    with torch.no_grad():
        pre = model(ids[:, :8], paged_cache=kv.bind(table, total_len=8))["logits"]
        assert torch.allclose(pre, dense[:, :8], atol=1e-5)
        for t in range(8, 11):   # ragged-mode decode steps
            pos = torch.full((2, 1), t)
            step = model(ids[:, t:t + 1], paged_cache=kv.bind(table, seq_lens=pos.squeeze(1) + 1), position_ids=pos)
            assert torch.allclose(step["logits"][:, 0], dense[:, t], atol=1e-4)
        # ragged multi-token step: sequence a has 5 cached positions, sequence b has 8; both add 3 tokens
        kv3 = KVCache(2, 16, 4, 2, 8, "cpu", torch.float32)
        for name in ("a", "b"):
            kv3.task_alloc(name, list(range(12)))
        ta, tb3 = kv3.make_table_tensor(["a"], "cpu"), kv3.make_table_tensor(["b"], "cpu")
        model(ids[:1, :5], paged_cache=kv3.bind(ta, total_len=5))
        model(ids[1:, :8], paged_cache=kv3.bind(tb3, total_len=8))
        both = kv3.make_table_tensor(["a", "b"], "cpu")
        new_ids = torch.stack([ids[0, 5:8], ids[1, 8:11]])
        pos = torch.stack([torch.arange(5, 8), torch.arange(8, 11)])
        rag = model(new_ids, paged_cache=kv3.bind(both, seq_lens=torch.tensor([8, 11])), position_ids=pos)["logits"]
        assert torch.allclose(rag[0], dense[0, 5:8], atol=1e-4) and torch.allclose(rag[1], dense[1, 8:11], atol=1e-4)
        # chunked prefill with a cached prefix (dense mode, start > 0)
        kv2 = KVCache(2, 16, 4, 2, 8, "cpu", torch.float32)
        kv2.task_alloc("a", list(range(12)))
        tb = kv2.make_table_tensor(["a"], "cpu")
        model(ids[:1, :4], paged_cache=kv2.bind(tb, total_len=4))
        pos = torch.arange(4, 11).unsqueeze(0)
        rest = model(ids[:1, 4:], paged_cache=kv2.bind(tb, total_len=11), position_ids=pos)["logits"]
        assert torch.allclose(rest, dense[:1, 4:], atol=1e-4)


# ---- tasks ----
def test_task_manager_state_machine(tokenizer):
    tm = TaskManager(tokenizer, max_batch_size=2, max_seq_len=32, max_prompt_len=8)
    seen = []
    tid = tm.add_task("hello world " * 40, stream_callback=seen.append)   # truncated to 8, fits
    assert tid.startswith("task_") and len(tm.get_waiting_tasks()[0].prompt_ids) == 8
    tm2 = TaskManager(tokenizer, max_batch_size=2, max_seq_len=4, max_prompt_len=8)
    tm2.add_task("hello world " * 40, stream_callback=seen.append)
    assert seen == [STOP] and tm2.get_waiting_tasks() == []              # too long: immediate STOP
    a = tm.add_task("hello", max_tokens=1000)
    b = tm.add_task([1, 2, 3], max_tokens=2)
    assert tm.get_waiting_tasks()[1].max_tokens == 32 - len(tm.get_waiting_tasks()[1].prompt_ids)
    first = tm.pull_candidates(2)
    assert [t.task_id for t in first] == [tid, a]                         # FIFO
    tm.return_to_waiting(first)
    assert [t.task_id for t in tm.get_waiting_tasks()] == [tid, a, b]
    t = tm.pull_candidates(1)[0]
    tm.activate(t)
    assert t.status == TaskStatus.RUNNING and tm.has_work()
    t.output_ids, t.output_tokens, t.max_tokens = [5, 6], 2, 2
    assert tm.remove_finished_tasks([]) == [t] and t.status == TaskStatus.FINISHED
    assert set(tm.get_stats()) >= {"total_tasks", "total_tokens", "active_tasks", "waiting_queue"}
    assert tm.get_stats()["total_tokens"] == 2
    tm.remove_task(a)
    assert [x.task_id for x in tm.get_waiting_tasks()] == [b]


# ---- sampling ----
def test_sampling_strategies():
    logits = torch.tensor([[1.0, 3.0, 2.0, 0.5], [0.1, 0.2, 4.0, 3.9]])
    assert torch.equal(TemperatureStrategy(1.0).apply(logits.clone()), logits)
    assert torch.equal(TopKStrategy(0).apply(logits.clone()), logits)
    assert torch.equal(TopPStrategy(1.0).apply(logits.clone()), logits)
    assert torch.allclose(TemperatureStrategy(torch.tensor([2.0, 0.5])).apply(logits.clone()), logits / torch.tensor([[2.0], [0.5]]))
    k = TopKStrategy(torch.tensor([1, 2])).apply(logits.clone())
    assert torch.isinf(k[0]).sum() == 3 and torch.isinf(k[1]).sum() == 2 and k[0, 1] == 3.0
    p0 = TopPStrategy(0.0).apply(logits.clone())
    assert torch.isinf(p0[0]).sum() == 3 and p0[0, 1] == 3.0
    nucleus = TopPStrategy(0.7).apply(torch.tensor([[0.0, 0.0, 10.0, 9.5]]))
    assert torch.isinf(nucleus[0, :2]).all() and not torch.isinf(nucleus[0, 2:]).any()
    torch.manual_seed(0)
    greedy = sample(logits.clone(), top_k=1)
    assert greedy.tolist() == [1, 2]
    draws = torch.stack([sample(logits.clone(), temperature=1.0, top_k=2) for _ in range(50)])
    assert set(draws[:, 0].tolist()) <= {1, 2} and set(draws[:, 1].tolist()) <= {2, 3}
    assert SamplingPipeline([TopKStrategy(1)]).sample(logits.clone()).tolist() == [1, 2]


# ---- engine ----
def test_generate_result_semantics():
    r = GenerateResult(count=2)
    r.append("a", 0); r.append("b", 1); r.append(STOP, 0); r.append(STOP, 0)
    assert r._completed == 1 and r.get_results() == ["a", "b"]
    assert [i for i, _ in r.pop_all()] == [0, 1, 0, 0] and r.pop_all() == []
    threading.Timer(0.05, lambda: r.append(STOP, 1)).start()
    r.wait_completion(timeout=2.0)
    with pytest.raises(TimeoutError):
        GenerateResult(1).wait_completion(timeout=0.05)


def test_generation_request_validation():
    GenerationRequest([{"role": "user", "content": "x"}], top_k=0, top_p=1.0, temperature=0.5)
    for kw, word in (({"top_k": -1}, "top_k"), ({"top_p": 1.5}, "top_p"), ({"temperature": 0}, "temperature")):
        with pytest.raises(ValueError, match=word):
            GenerationRequest([], **kw)


@pytest.fixture
def engine(tokenizer):
    torch.manual_seed(0)
    model = AutoRegressiveLM(tiny_config(vocab_size=len(tokenizer))).eval()
    with InferenceEngine(model, tokenizer, max_batch_size=3, max_seq_len=64, page_size=4) as eng:
        yield eng


def _dense_greedy(model, tokenizer, prompt, n):
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


def test_engine_ragged_batch_matches_dense_greedy(engine, tokenizer):
    prompts = ["hello world", "the quick brown fox jumps over", "a", "this is a test", "hello world"]
    got = engine.generate(prompts, max_tokens=8, top_k=1)
    assert isinstance(got, list) and len(got) == 5
    for p, text in zip(prompts, got):
        assert text == _dense_greedy(engine.model, tokenizer, p, 8)
    assert isinstance(engine.generate("hello", max_tokens=3, top_k=1), str)
    stats = engine.get_stats()
    assert stats["total_tasks"] == 6 and stats["active_tasks"] == 0 and stats["ttft_p50_s"] is not None
    hist = engine.get_histograms()
    assert hist["latency_seconds"]["count"] == 6 and hist["ttft_seconds"]["count"] == 6
    assert hist["latency_seconds"]["sum"] >= hist["ttft_seconds"]["sum"] > 0


def test_engine_streaming_async_and_request(engine, tokenizer):
    import asyncio

    toks = list(engine.generate("hello world", stream=True, max_tokens=5, top_k=1))
    assert "".join(toks) == _dense_greedy(engine.model, tokenizer, "hello world", 5)
    pairs = list(engine.generate(["hello", "world"], stream=True, max_tokens=3, top_k=1))
    assert {i for i, _ in pairs} <= {0, 1} and all(isinstance(t, str) for _, t in pairs)

    async def collect():
        return [t async for t in engine.generate_async("hello world", max_tokens=5, top_k=1)]

    assert asyncio.run(collect()) == toks
    req = GenerationRequest([{"role": "user", "content": "hello"}], top_k=1, max_tokens=4)
    assert isinstance(engine.generate_with_request(req), str)


def test_scheduler_thread_safety_and_page_release(engine):
    errors = []

    def worker(i):
        try:
            for _ in range(3):
                engine.generate(f"hello {i}", max_tokens=4, top_k=1)
                engine.get_stats()
        except Exception as exc:  # pragma: no cover
            errors.append(exc)

    threads = [threading.Thread(target=worker, args=(i,)) for i in range(6)]
    [t.start() for t in threads]
    [t.join(timeout=60) for t in threads]
    assert not errors and engine.get_stats()["total_tasks"] == 18
    time.sleep(0.1)
    sched = engine.scheduler
    assert sched._page_cache.free_pages() == sched._page_cache._storage.n_pages   # everything returned


def test_scheduler_fatal_error_drains_tasks(tokenizer):
    class Broken(AutoRegressiveLM):
        def forward(self, *a, **k):
            raise RuntimeError("boom")

    eng = InferenceEngine(Broken(tiny_config(vocab_size=len(tokenizer))), tokenizer, max_batch_size=2, max_seq_len=32,
                          page_size=4)
    assert eng.generate("hello", max_tokens=4) == ""          # STOP delivered instead of hanging
    assert isinstance(eng.scheduler._fatal_error, RuntimeError)
    eng.shutdown()


def test_kv_exhaustion_aborts_instead_of_hanging(tokenizer):
    model = AutoRegressiveLM(tiny_config(vocab_size=len(tokenizer))).eval()
    eng = InferenceEngine(model, tokenizer, max_batch_size=1, max_seq_len=16, page_size=4)
    # steal all but two pages: the prompt fits, growth does not
    cache = eng.scheduler._page_cache
    while cache.free_pages() > 2:
        cache._pool.alloc()
    t0 = time.time()
    out = eng.generate("hello world this is a test", max_tokens=12, top_k=1)
    assert time.time() - t0 < 20 and isinstance(out, str)
    eng.shutdown()


def test_split_kv_factor_fills_whole_waves():
    from khaosz_b200.inference.core.cache import _pick_splits

    assert _pick_splits(1024, 2048) == 1            # already many CTAs per SM
    n = _pick_splits(256, 2048)                     # 256 CTAs on 148 SMs: 1.7 waves -> split
    assert n > 1 and (256 * n) % 148 <= 148 and -(-256 * n // 148) * 148 / (256 * n) < 1.1
    assert _pick_splits(4, 128) == 1                # a single 128-key tile cannot be split
    assert 1 <= _pick_splits(4, 4096) <= 16
