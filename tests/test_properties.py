"""Property-based checks (hypothesis) of the pieces whose correctness is an invariant rather than an
example: segmented store reads, dataset windows, the sampler's partition of an epoch, the page
allocator's bookkeeping, the prefix index, stop-sequence handling and top-k / top-p filtering."""
import tempfile

import torch
from hypothesis import given, settings
from hypothesis import strategies as st

from khaosz_b200.data import DatasetFactory, MmapStore, ResumableDistributedSampler, save_bin
from khaosz_b200.inference import Allocator, KVCache, PrefixCache, TopKStrategy, TopPStrategy
from khaosz_b200.inference.api import AnthropicResponseBuilder, StopChecker, StopInfo
from khaosz_b200.inference.api.protocol import GenContext

FAST = settings(max_examples=60, deadline=None)


@FAST
@given(st.lists(st.integers(1, 12), min_size=1, max_size=6), st.data())
def test_store_reads_equal_slices_of_the_concatenation(segment_lengths, data):
    store = MmapStore()
    pieces, start = [], 0
    for n in segment_lengths:
        pieces.append(torch.arange(start, start + n))
        start += n
    store._install({"sequence": pieces})
    whole = torch.cat(pieces)
    begin = data.draw(st.integers(0, len(whole) - 1))
    end = data.draw(st.integers(begin, len(whole)))
    assert torch.equal(store.fetch(begin, end, "sequence"), whole[begin:end])


@FAST
@given(st.integers(2, 120), st.integers(1, 16), st.integers(1, 20))
def test_dataset_windows_stay_inside_the_data_and_cover_it(total, window, stride):
    with tempfile.TemporaryDirectory() as tmp:
        save_bin(tmp, {"sequence": [torch.arange(total, dtype=torch.int32)]})
        ds = DatasetFactory.load("seq", tmp, window, stride)
        assert len(ds) == (0 if total <= window else (total - 1 - window) // stride + 1)
        for i in range(len(ds)):
            item = ds[i]
            assert item["input_ids"].shape == (window,) and int(item["target_ids"][-1]) <= total - 1
            assert torch.equal(item["target_ids"], item["input_ids"] + 1)
            assert int(item["input_ids"][0]) == min(i * stride, total - 1 - window)
        del ds


@FAST
@given(st.integers(1, 60), st.integers(1, 7), st.integers(0, 10 ** 6), st.integers(0, 5))
def test_sampler_shares_partition_the_padded_epoch(n, replicas, seed, epoch):
    shares = [list(ResumableDistributedSampler(range(n), seed=seed, start_epoch=epoch, num_replicas=replicas, rank=r))
              for r in range(replicas)]
    per_rank = -(-n // replicas)
    assert all(len(s) == per_rank for s in shares)
    seen = [i for s in shares for i in s]
    assert set(seen) == set(range(n)) and len(seen) == per_rank * replicas
    again = list(ResumableDistributedSampler(range(n), seed=seed, start_epoch=epoch, num_replicas=replicas, rank=0))
    assert again == shares[0]


@FAST
@given(st.integers(1, 40), st.integers(1, 4), st.data())
def test_sampler_resume_yields_the_rest_of_the_epoch(n, replicas, data):
    rank = data.draw(st.integers(0, replicas - 1))
    whole = list(ResumableDistributedSampler(range(n), seed=3, num_replicas=replicas, rank=rank))
    skip = data.draw(st.integers(0, len(whole)))
    resumed = list(ResumableDistributedSampler(range(n), seed=3, start_iter=skip, num_replicas=replicas, rank=rank))
    assert resumed == whole[skip:]


@FAST
@given(st.integers(1, 8), st.lists(st.tuples(st.sampled_from(["alloc", "free", "park", "share"]), st.integers(0, 7)), max_size=60))
def test_allocator_never_loses_or_duplicates_a_page(n_pages, script):
    a = Allocator(n_pages)
    owned = {}                                          # page -> number of references we hold
    for op, arg in script:
        if op == "alloc":
            p = a.alloc()
            if p >= 0:
                assert p not in owned and 0 <= p < n_pages
                owned[p] = 1
            else:
                assert len(owned) == n_pages            # -1 only when everything is in use
        elif owned:
            p = sorted(owned)[arg % len(owned)]
            if op == "share":
                a.inc_ref(p)
                owned[p] += 1
            else:
                a.free(p, keep_cached=(op == "park"))
                owned[p] -= 1
                if owned[p] == 0:
                    del owned[p]
        assert a.free_pages() == n_pages - len(owned)
        assert all(a.ref_count(p) == c for p, c in owned.items())


@FAST
@given(st.lists(st.integers(0, 5), min_size=0, max_size=24), st.lists(st.integers(0, 5), min_size=0, max_size=24),
       st.integers(1, 4))
def test_prefix_hits_are_exactly_the_common_full_pages(first, second, page_size):
    pc = PrefixCache(page_size)
    for logical in range(len(first) // page_size):
        pc.record(100 + logical, first, logical)
    common = 0
    while common < min(len(first), len(second)) and first[common] == second[common]:
        common += 1
    expected_pages = min(common // page_size, len(first) // page_size)
    assert pc.lookup(second) == [100 + i for i in range(expected_pages)]


@FAST
@given(st.lists(st.lists(st.integers(0, 3), min_size=1, max_size=14), min_size=1, max_size=6), st.integers(1, 4))
def test_kv_accounting_returns_every_page(prompts, page_size):
    total = sum(-(-len(p) // page_size) for p in prompts) + 2
    kv = KVCache(1, total, page_size, 1, 4, "cpu", torch.float32)
    for i, prompt in enumerate(prompts):
        assert kv.task_alloc(f"t{i}", prompt)
        kv.task_record_hashes(f"t{i}", prompt)
        table = kv._table.get(f"t{i}")
        assert len(table) == -(-len(prompt) // page_size) and kv.task_cached(f"t{i}") % page_size == 0
        assert kv.task_cached(f"t{i}") <= len(prompt)
    for i in range(len(prompts)):
        kv.task_free(f"t{i}")
    assert kv.free_pages() == total


@FAST
@given(st.text(alphabet="abcX", max_size=30), st.lists(st.text(alphabet="abcX", min_size=1, max_size=3), max_size=3))
def test_stop_checker_agrees_with_substring_search(text, stops):
    found = StopChecker(stops).check(text)
    if any(s in text for s in stops):
        assert found == next(s for s in stops if s in text)
    else:
        assert found is None


@FAST
@given(st.text(alphabet="ab ", max_size=12), st.text(alphabet="ab ", max_size=6), st.integers(0, 12))
def test_anthropic_stream_never_repeats_or_drops_text_before_the_stop(before, after, sent):
    body = before + "END" + after
    yielded = before[:min(sent, len(before))]
    events = AnthropicResponseBuilder().format_stream_end(GenContext("m", 0, "x", 1, 1), StopInfo("END", body, yielded))
    flushed = "".join(e.split('"text": "')[1].split('"}')[0] for e in events if "content_block_delta" in e.split("\n")[0])
    assert yielded + flushed.encode().decode("unicode_escape") == body[:body.rfind("END")]


@FAST
@given(st.lists(st.floats(-8, 8, allow_nan=False), min_size=2, max_size=12), st.integers(0, 14), st.floats(0.0, 1.0))
def test_filters_keep_the_argmax_and_only_remove(values, k, p):
    logits = torch.tensor([values])
    for out in (TopKStrategy(k).apply(logits.clone()), TopPStrategy(p).apply(logits.clone())):
        kept = ~torch.isinf(out)
        assert kept[0, logits.argmax()]                                   # the most likely token always survives
        assert torch.equal(out[kept], logits[kept])                       # survivors are untouched
    top = TopKStrategy(k).apply(logits.clone())
    if 0 < k < len(values):
        assert int((~torch.isinf(top)).sum()) >= k                        # ties may keep more, never fewer


def test_fp8_quantisers_and_input_gradient_oracle_on_cpu():
    """The CPU forms of the block-scaled fp8 quantisers are the oracles of the GPU kernels: the input gradient
    built from them (output gradient with 1x128 scales, transposed weight with 128x128 scales) reproduces the
    fp32 product to fp8 accuracy, and the transposed weight image is cached per weight generation."""
    import torch

    from khaosz_b200.ops import functional as Fn
    from khaosz_b200.ops import quant

    torch.manual_seed(0)
    M, K, N = 256, 512, 384
    dy = torch.randn(M, N).to(torch.bfloat16)
    w = (torch.randn(N, K) * 0.05).to(torch.bfloat16)
    ref = dy.float() @ w.float()
    dx = Fn.dgrad_fp8(dy, w)
    assert dx.shape == (M, K) and dx.dtype == torch.bfloat16
    assert (dx.float() - ref).abs().mean().item() <= 0.06 * ref.abs().mean().item()
    w8, sw = Fn._fp8_weight_t(w)
    assert w8.shape == (K, N) and sw.shape == (K // 128, N // 128)
    assert Fn._fp8_weight_t(w)[0] is w8                       # cached ...
    Fn.bump_weight_generation()
    assert Fn._fp8_weight_t(w)[0] is not w8                   # ... for one weight generation
    back = quant.dequantize_fp8(w8, sw, True)
    assert (back - w.float().t()).abs().max().item() <= 0.07 * w.float().abs().max().item()


def test_fp8_weight_cache_is_not_fooled_by_a_reused_address():
    """The fp8 weight images are found by address; an entry keeps its weight alive, so a tensor that is freed
    within a weight generation cannot hand its address (and its stale image) to the next weight."""
    import torch

    from khaosz_b200.ops import functional as Fn
    from khaosz_b200.ops import quant

    torch.manual_seed(1)
    for _ in range(4):                       # allocate / free the same size repeatedly: the allocator reuses blocks
        w = (torch.randn(256, 256) * torch.rand(()).item()).to(torch.bfloat16)
        for cached, fresh in ((Fn._fp8_weight(w), quant.quantize_fp8_128x128(w)),
                              (Fn._fp8_weight_t(w), quant.quantize_fp8_128x128(w.t().contiguous()))):
            assert torch.equal(cached[0], fresh[0]) and torch.equal(cached[1], fresh[1])
        del w
    Fn.bump_weight_generation()
    assert not Fn._FP8_WEIGHT_CACHE
