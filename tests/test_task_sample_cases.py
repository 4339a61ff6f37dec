"""Case-by-case behaviour of generation tasks, the task manager and the sampling strategies (the
behaviours the reference pins in ``tests/inference/test_task.py`` and ``tests/inference/test_sample.py``)."""
import threading
import time

import pytest
import torch

from khaosz_b200.inference import (STOP, SamplingPipeline, TaskManager, TaskStatus, TemperatureStrategy, TopKStrategy,
                                   TopPStrategy, sample)
from khaosz_b200.inference.core.task import Histogram, Task


class _Words:
    """One token per word; ids are the word lengths."""

    def encode(self, text, **_):
        return [len(w) for w in text.split()]


def _manager(**kw):
    args = dict(max_batch_size=4, max_seq_len=32, max_prompt_len=16)
    args.update(kw)
    return TaskManager(_Words(), **args)


# ---- Task -------------------------------------------------------------------------------------
def test_new_task_is_pending_with_no_output():
    t = Task("task_x", [1, 2, 3], max_tokens=5)
    assert t.status == TaskStatus.PENDING and t.output_ids == [] and t.output_tokens == 0
    assert t.first_token_time is None and t.finish_time is None and t.arrival_time <= time.time()
    assert (t.temperature, t.top_p, t.top_k) == (1.0, 1.0, 50)


def test_next_pos_counts_prefilled_and_generated_tokens():
    t = Task("task_x", [1, 2, 3])
    assert t.next_pos == 0                              # nothing in the cache yet
    t.input_tokens = 3
    assert t.next_pos == 3
    t.output_ids += [7, 8]
    assert t.next_pos == 5


def test_task_finishes_at_max_tokens():
    t = Task("task_x", [1], max_tokens=2)
    t.output_ids, t.output_tokens = [4], 1
    assert not t.is_finished([])
    t.output_ids, t.output_tokens = [4, 5], 2
    assert t.is_finished([])


def test_task_finishes_on_a_stop_token_only_when_it_is_the_last_one():
    t = Task("task_x", [1], max_tokens=10)
    assert not t.is_finished([9])                       # no output yet
    t.output_ids, t.output_tokens = [9, 4], 2
    assert not t.is_finished([9])
    t.output_ids, t.output_tokens = [9, 4, 9], 3
    assert t.is_finished([9]) and t.is_finished([3, 9])


def test_task_without_max_tokens_runs_until_a_stop_token():
    t = Task("task_x", [1], max_tokens=None)
    t.output_ids, t.output_tokens = list(range(1000)), 1000
    assert not t.is_finished([5000]) and t.is_finished([999])


# ---- TaskManager ------------------------------------------------------------------------------
def test_add_task_queues_a_pending_task_with_a_fresh_id():
    tm = _manager()
    a, b = tm.add_task("aa bbb c"), tm.add_task("dddd")
    assert a.startswith("task_") and b.startswith("task_") and a != b
    waiting = tm.get_waiting_tasks()
    assert [t.task_id for t in waiting] == [a, b] and waiting[0].prompt_ids == [2, 3, 1]
    assert waiting[0].status == TaskStatus.PENDING and tm.get_active_tasks() == []


def test_add_task_accepts_token_ids():
    tm = _manager()
    tm.add_task([5, 6, 7])
    tm.add_task((8, 9))
    assert [t.prompt_ids for t in tm.get_waiting_tasks()] == [[5, 6, 7], [8, 9]]


def test_add_task_keeps_the_sampling_parameters():
    tm = _manager()
    tm.add_task("a", max_tokens=3, temperature=0.5, top_p=0.9, top_k=7)
    t = tm.get_waiting_tasks()[0]
    assert (t.max_tokens, t.temperature, t.top_p, t.top_k) == (3, 0.5, 0.9, 7)


def test_long_prompts_keep_their_tail():
    tm = _manager(max_prompt_len=4)
    tm.add_task([1, 2, 3, 4, 5, 6, 7])
    assert tm.get_waiting_tasks()[0].prompt_ids == [4, 5, 6, 7]


def test_max_tokens_is_clamped_to_the_room_left():
    tm = _manager(max_seq_len=10)
    tm.add_task([1] * 6, max_tokens=100)
    tm.add_task([1] * 6)
    tm.add_task([1] * 6, max_tokens=2)
    assert [t.max_tokens for t in tm.get_waiting_tasks()] == [4, 4, 2]


def test_prompt_that_fills_the_sequence_stops_at_once():
    tm = _manager(max_seq_len=4, max_prompt_len=8)
    seen = []
    tid = tm.add_task([1] * 6, stream_callback=seen.append)
    assert tid.startswith("task_") and seen == [STOP]
    assert tm.get_waiting_tasks() == [] and not tm.has_work() and tm.get_stats()["total_tasks"] == 0
    tm.add_task([1] * 6)                                # without a callback it is dropped silently


def test_pull_candidates_is_first_in_first_out_and_bounded():
    tm = _manager()
    ids = [tm.add_task([i + 1]) for i in range(3)]
    assert tm.pull_candidates(0) == [] and tm.pull_candidates(-3) == []
    assert [t.task_id for t in tm.pull_candidates(2)] == ids[:2]
    assert [t.task_id for t in tm.pull_candidates(5)] == ids[2:]
    assert tm.pull_candidates(1) == []


def test_activate_marks_running():
    tm = _manager()
    tm.add_task([1])
    t = tm.pull_candidates(1)[0]
    tm.activate(t)
    assert t.status == TaskStatus.RUNNING and tm.get_active_tasks() == [t] and tm.get_waiting_tasks() == []


def test_return_to_waiting_puts_tasks_back_at_the_head_in_order():
    tm = _manager()
    ids = [tm.add_task([i + 1]) for i in range(4)]
    pulled = tm.pull_candidates(2)
    tm.return_to_waiting(pulled)
    assert [t.task_id for t in tm.get_waiting_tasks()] == ids


def test_remove_task_from_the_queue_and_from_the_batch():
    tm = _manager()
    a, b = tm.add_task([1]), tm.add_task([2])
    assert tm.remove_task(a) == []                      # was only waiting: nothing whose pages need freeing
    t = tm.pull_candidates(1)[0]
    tm.activate(t)
    assert tm.remove_task(b) == [t] and not tm.has_work()
    assert tm.remove_task("task_unknown") == []


def test_remove_finished_collects_aborted_tasks():
    tm = _manager()
    tm.add_task([1])
    t = tm.pull_candidates(1)[0]
    tm.activate(t)
    t.status = TaskStatus.ABORTED
    assert tm.remove_finished_tasks([]) == [t] and t.finish_time is not None
    assert tm.get_active_tasks() == [] and tm.get_stats()["total_tokens"] == 0


def test_remove_finished_on_stop_token_counts_the_tokens():
    tm = _manager()
    tm.add_task([1], max_tokens=10)
    tm.add_task([2], max_tokens=10)
    done, running = tm.pull_candidates(2)
    tm.activate(done)
    tm.activate(running)
    done.output_ids, done.output_tokens, done.first_token_time = [4, 99], 2, time.time()
    running.output_ids, running.output_tokens = [4], 1
    assert tm.remove_finished_tasks([99]) == [done]
    assert done.status == TaskStatus.FINISHED and tm.get_active_tasks() == [running]
    assert tm.get_stats()["total_tokens"] == 2 and tm.latency_stats()["finished"] == 1
    assert tm.remove_finished_tasks([99]) == []


def test_has_work_covers_queue_and_batch():
    tm = _manager()
    assert not tm.has_work()
    tm.add_task([1])
    assert tm.has_work()
    t = tm.pull_candidates(1)[0]
    assert not tm.has_work()                            # pulled but not yet activated
    tm.activate(t)
    assert tm.has_work()
    tm.clear_queues()
    assert not tm.has_work()


def test_wait_for_tasks_returns_when_work_arrives_or_on_wake():
    tm = _manager()
    start = time.time()
    tm.wait_for_tasks(timeout=0.05)
    assert time.time() - start >= 0.04                  # nothing to do: waits out the timeout
    threading.Timer(0.05, tm.wake).start()
    start = time.time()
    tm.wait_for_tasks(timeout=5.0)
    assert time.time() - start < 2.0
    tm.add_task([1])
    start = time.time()
    tm.wait_for_tasks(timeout=5.0)                      # work is queued: no wait at all
    assert time.time() - start < 0.5


def test_stats_keys_and_counts():
    tm = _manager()
    assert tm.get_stats() == {"total_tasks": 0, "total_tokens": 0, "active_tasks": 0, "waiting_queue": 0}
    tm.add_task([1])
    tm.add_task([2])
    tm.activate(tm.pull_candidates(1)[0])
    assert tm.get_stats() == {"total_tasks": 2, "total_tokens": 0, "active_tasks": 1, "waiting_queue": 1}
    lat = tm.latency_stats()
    assert lat["finished"] == 0 and lat["ttft_p50_s"] is None and lat["itl_p99_s"] is None


def test_latency_statistics_of_finished_requests():
    tm = _manager()
    tm.add_task([1], max_tokens=3)
    t = tm.pull_candidates(1)[0]
    tm.activate(t)
    t.arrival_time = time.time() - 1.0
    t.first_token_time = t.arrival_time + 0.25
    t.output_ids, t.output_tokens = [1, 2, 3], 3
    tm.remove_finished_tasks([])
    lat = tm.latency_stats()
    assert lat["ttft_p50_s"] == pytest.approx(0.25, abs=1e-6) and lat["latency_p50_s"] == pytest.approx(1.0, abs=0.1)
    assert lat["itl_p50_s"] == pytest.approx(0.375, abs=0.05)             # (1.0 - 0.25) / 2 gaps
    hist = tm.histograms()
    assert hist["ttft_seconds"]["count"] == hist["itl_seconds"]["count"] == hist["latency_seconds"]["count"] == 1
    assert hist["ttft_seconds"]["cumulative"][hist["ttft_seconds"]["bounds"].index(0.25)] == 1


def test_histogram_buckets_are_cumulative():
    h = Histogram(bounds=(1.0, 2.0, 4.0))
    for v in (0.5, 1.0, 1.5, 3.0, 9.0):
        h.observe(v)
    snap = h.snapshot()
    assert snap["cumulative"] == [2, 3, 4] and snap["count"] == 5 and snap["sum"] == pytest.approx(15.0)


# ---- sampling ---------------------------------------------------------------------------------
LOGITS = torch.tensor([[1.0, 3.0, 2.0, 0.5], [0.1, 0.2, 4.0, 3.9]])


def test_temperature_divides_the_logits():
    assert torch.allclose(TemperatureStrategy(2.0).apply(LOGITS.clone()), LOGITS / 2.0)
    assert torch.allclose(TemperatureStrategy(0.5).apply(LOGITS.clone()), LOGITS * 2.0)


def test_temperature_one_is_an_exact_no_op():
    assert torch.equal(TemperatureStrategy(1.0).apply(LOGITS.clone()), LOGITS)
    assert torch.equal(TemperatureStrategy().apply(LOGITS.clone()), LOGITS)


def test_temperature_per_row_and_near_zero():
    out = TemperatureStrategy(torch.tensor([2.0, 0.5])).apply(LOGITS.clone())
    assert torch.allclose(out[0], LOGITS[0] / 2.0) and torch.allclose(out[1], LOGITS[1] / 0.5)
    tiny = TemperatureStrategy(0.0).apply(LOGITS.clone())              # clamped, not a division by zero
    assert torch.isfinite(tiny).all() and tiny.argmax(dim=-1).tolist() == [1, 2]


def test_top_k_keeps_the_k_largest():
    out = TopKStrategy(2).apply(LOGITS.clone())
    assert torch.isinf(out).sum(dim=-1).tolist() == [2, 2]
    assert out[0, 1] == 3.0 and out[0, 2] == 2.0 and out[1, 2] == 4.0 and out[1, 3] == pytest.approx(3.9)


def test_top_k_zero_and_oversized_k_change_nothing():
    assert torch.equal(TopKStrategy(0).apply(LOGITS.clone()), LOGITS)
    assert torch.equal(TopKStrategy(100).apply(LOGITS.clone()), LOGITS)


def test_top_k_per_row():
    out = TopKStrategy(torch.tensor([1, 3])).apply(LOGITS.clone())
    assert torch.isinf(out).sum(dim=-1).tolist() == [3, 1] and out[0, 1] == 3.0 and torch.isinf(out[1, 0])
    mixed = TopKStrategy(torch.tensor([0, 1])).apply(LOGITS.clone())    # 0 = off for that row
    assert torch.equal(mixed[0], LOGITS[0]) and torch.isinf(mixed[1]).sum() == 3


def test_top_p_keeps_the_smallest_set_reaching_p():
    logits = torch.tensor([[0.0, 0.0, 10.0, 9.5]])                      # probabilities about 0.62 / 0.38 / ~0 / ~0
    assert torch.isinf(TopPStrategy(0.5).apply(logits.clone())).tolist() == [[True, True, False, True]]
    assert torch.isinf(TopPStrategy(0.7).apply(logits.clone())).tolist() == [[True, True, False, False]]


def test_top_p_one_is_an_exact_no_op_and_zero_keeps_the_maximum():
    assert torch.equal(TopPStrategy(1.0).apply(LOGITS.clone()), LOGITS)
    out = TopPStrategy(0.0).apply(LOGITS.clone())
    assert torch.isinf(out).sum(dim=-1).tolist() == [3, 3] and out[0, 1] == 3.0 and out[1, 2] == 4.0


def test_top_p_per_row():
    logits = torch.tensor([[0.0, 0.0, 10.0, 9.5], [0.0, 0.0, 10.0, 9.5]])
    out = TopPStrategy(torch.tensor([0.5, 1.0])).apply(logits.clone())
    assert torch.isinf(out[0]).sum() == 3 and torch.equal(out[1], logits[1])


def test_filter_value_can_be_chosen():
    out = TopKStrategy(1).apply(LOGITS.clone(), filter_value=-1e4)
    assert (out == -1e4).sum() == 6 and not torch.isinf(out).any()


def test_pipeline_applies_its_strategies_in_order():
    pipe = SamplingPipeline([TemperatureStrategy(0.5), TopKStrategy(2), TopPStrategy(0.99)])
    out = pipe.apply(LOGITS.clone())
    assert out[0, 1] == 6.0 and torch.isinf(out[0, 0]) and torch.isinf(out[0, 3])
    assert torch.equal(SamplingPipeline([]).apply(LOGITS.clone()), LOGITS)


def test_pipeline_sample_returns_one_valid_token_per_row():
    torch.manual_seed(0)
    pipe = SamplingPipeline([TopKStrategy(2)])
    draws = torch.stack([pipe.sample(LOGITS.clone()) for _ in range(40)])
    assert draws.shape == (40, 2) and draws.dtype == torch.long
    assert set(draws[:, 0].tolist()) <= {1, 2} and set(draws[:, 1].tolist()) <= {2, 3}


def test_sample_shortcut_is_greedy_with_top_k_one():
    assert sample(LOGITS.clone(), top_k=1).tolist() == [1, 2]
    assert sample(LOGITS[0].clone().unsqueeze(0), temperature=0.7, top_k=1, top_p=0.5).tolist() == [1]


def test_sample_follows_the_distribution():
    torch.manual_seed(0)
    logits = torch.log(torch.tensor([[0.7, 0.2, 0.1]])).repeat(4000, 1)
    freq = torch.bincount(sample(logits), minlength=3).float() / 4000
    assert freq.tolist() == pytest.approx([0.7, 0.2, 0.1], abs=0.03)


def test_sample_with_per_row_parameters():
    torch.manual_seed(0)
    logits = LOGITS.repeat(50, 1)                                       # rows alternate between the two patterns
    k = torch.tensor([1, 2] * 50)
    out = sample(logits, temperature=torch.tensor([1.0, 0.5] * 50), top_k=k, top_p=torch.tensor([1.0, 0.9] * 50))
    assert set(out[0::2].tolist()) == {1} and set(out[1::2].tolist()) <= {2, 3}


def test_cancel_withdraws_waiting_tasks_and_only_marks_running_ones():
    tm = _manager()
    a, b = tm.add_task([1]), tm.add_task([2])
    running = tm.pull_candidates(1)[0]
    tm.activate(running)
    gone = tm.cancel(b)
    assert gone.task_id == b and gone.status == TaskStatus.ABORTED and tm.get_waiting_tasks() == []
    marked = tm.cancel(a)
    assert marked is running and running.status == TaskStatus.ABORTED
    assert tm.get_active_tasks() == [running]           # still listed: the scheduler thread frees its pages
    assert tm.remove_finished_tasks([]) == [running] and tm.get_active_tasks() == []
    assert tm.cancel(a) is None and tm.cancel("task_unknown") is None


def test_cancel_reaches_a_task_that_is_being_admitted():
    tm = _manager()
    tid = tm.add_task([1])
    pulled = tm.pull_candidates(1)[0]                   # neither waiting nor active at this moment
    assert tm.cancel(tid) is None
    tm.activate(pulled)
    assert pulled.status == TaskStatus.ABORTED and tm.remove_finished_tasks([]) == [pulled]
    other = tm.add_task([2])
    fresh = tm.pull_candidates(1)[0]
    tm.activate(fresh)
    assert fresh.status == TaskStatus.RUNNING and other == fresh.task_id


def test_cancelled_ids_do_not_pile_up():
    tm = _manager()
    for i in range(5000):
        tm.cancel(f"task_gone_{i}")
    assert len(tm._cancelled) <= 1024


def test_empty_prompts_and_zero_budgets_are_closed_without_queueing():
    tm = _manager()
    seen = []
    tm.add_task([], stream_callback=seen.append)
    tm.add_task("", stream_callback=seen.append)
    tm.add_task([1, 2], max_tokens=0, stream_callback=seen.append)
    assert seen == [STOP, STOP, STOP] and tm.get_waiting_tasks() == [] and tm.get_stats()["total_tasks"] == 0


def test_rows_with_nan_or_infinite_logits_do_not_fail_the_batch():
    torch.manual_seed(0)
    logits = torch.randn(3, 20)
    logits[0, 7] = float("inf")
    logits[1, 2] = float("nan")
    out = sample(logits)
    assert out[0] == 7 and out[1] == logits[1].nan_to_num(nan=float("-inf")).argmax() and 0 <= int(out[2]) < 20
