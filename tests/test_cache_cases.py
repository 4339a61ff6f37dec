"""Case-by-case behaviour of the paged KV cache: page hash, allocator, prefix index, page pool, task
table, K/V storage and the per-task accounting (the behaviours the reference pins in
``tests/inference/test_cache.py``, plus the chained prefix hash this cache uses)."""
import threading

import torch

from khaosz_b200.inference import Allocator, KVCache, PagePool, PrefixCache, Storage, TaskTable, page_hash


# ---- page hash --------------------------------------------------------------------------------
def test_page_hash_is_deterministic_and_fits_64_bits():
    toks = list(range(100, 132))
    assert page_hash(toks, 0, 16) == page_hash(list(toks), 0, 16)
    assert 0 <= page_hash(toks, 1, 16) < 2 ** 64


def test_page_hash_depends_on_content_and_order():
    assert page_hash([1, 2, 3, 4], 0, 4) != page_hash([1, 2, 3, 5], 0, 4)
    assert page_hash([1, 2, 3, 4], 0, 4) != page_hash([4, 3, 2, 1], 0, 4)
    assert page_hash([0, 0], 0, 4) != page_hash([0], 0, 4)                      # token 0 still counts


def test_page_hash_is_chained_over_the_prefix():
    a, b = [1, 2, 3, 4, 9, 9, 9, 9], [5, 6, 7, 8, 9, 9, 9, 9]
    assert page_hash(a, 1, 4) != page_hash(b, 1, 4)                              # same second page, other first page
    assert page_hash(a, 0, 4) == page_hash(a[:4] + [0, 0, 0, 0], 0, 4)           # page 0 ignores what follows


# ---- allocator --------------------------------------------------------------------------------
def test_allocator_hands_out_every_page_once_then_minus_one():
    a = Allocator(4)
    assert a.free_pages() == 4
    got = [a.alloc() for _ in range(4)]
    assert sorted(got) == [0, 1, 2, 3] and all(a.ref_count(p) == 1 for p in got)
    assert a.alloc() == -1 and a.free_pages() == 0


def test_allocator_free_then_alloc_reuses_the_page():
    a = Allocator(2)
    p, q = a.alloc(), a.alloc()
    a.free(p)
    assert a.free_pages() == 1 and a.ref_count(p) == 0
    assert a.alloc() == p and a.alloc() == -1
    a.free(q)
    assert a.alloc() == q


def test_allocator_shared_page_needs_every_owner_to_let_go():
    a = Allocator(1)
    p = a.alloc()
    a.inc_ref(p)
    a.inc_ref(p)
    assert a.ref_count(p) == 3
    a.free(p)
    a.free(p)
    assert a.alloc() == -1 and a.ref_count(p) == 1
    a.free(p)
    assert a.alloc() == p


def test_allocator_prefers_free_pages_over_cached_ones():
    a = Allocator(3)
    p0, p1, p2 = a.alloc(), a.alloc(), a.alloc()
    evicted = []
    a.on_evict = evicted.append
    a.free(p0, keep_cached=True)
    a.free(p1)
    assert a.free_pages() == 2
    assert a.alloc() == p1 and evicted == []
    assert a.alloc() == p0 and evicted == [p0]
    assert a.alloc() == -1


def test_allocator_evicts_least_recently_used_first_and_touch_refreshes():
    a = Allocator(3)
    pages = [a.alloc() for _ in range(3)]
    for p in pages:
        a.free(p, keep_cached=True)
    a.touch(pages[0])                                   # now the most recently used
    evicted = []
    a.on_evict = evicted.append
    assert [a.alloc(), a.alloc(), a.alloc()] == [pages[1], pages[2], pages[0]]
    assert evicted == [pages[1], pages[2], pages[0]]


def test_allocator_reviving_a_cached_page_takes_it_out_of_the_lru():
    a = Allocator(2)
    p, q = a.alloc(), a.alloc()
    a.free(p, keep_cached=True)
    a.inc_ref(p)                                        # a new task found it through the prefix index
    a.free(q)
    assert a.alloc() == q and a.alloc() == -1           # p is in use again: not a victim
    assert a.ref_count(p) == 1


def test_allocator_is_thread_safe():
    a = Allocator(64)
    got, lock = [], threading.Lock()

    def worker():
        mine = [a.alloc() for _ in range(8)]
        with lock:
            got.extend(mine)

    threads = [threading.Thread(target=worker) for _ in range(8)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    assert sorted(got) == list(range(64))


# ---- prefix index -----------------------------------------------------------------------------
def test_prefix_lookup_returns_the_recorded_pages_in_order():
    pc = PrefixCache(4)
    toks = list(range(12))
    for logical, page in enumerate([5, 3, 8]):
        pc.record(page, toks, logical)
    assert pc.lookup(toks) == [5, 3, 8] and pc.lookup(toks[:8]) == [5, 3] and pc.lookup(toks[:7]) == [5]


def test_prefix_lookup_stops_at_the_first_miss():
    pc = PrefixCache(4)
    toks = list(range(12))
    pc.record(1, toks, 0)
    pc.record(2, toks, 2)                                # page 1 of the prompt was never recorded
    assert pc.lookup(toks) == [1]


def test_prefix_lookup_ignores_a_partial_last_page_and_short_prompts():
    pc = PrefixCache(4)
    pc.record(0, [1, 2, 3, 4], 0)
    assert pc.lookup([1, 2, 3, 4, 5, 6]) == [0]
    assert pc.lookup([1, 2, 3]) == [] and pc.lookup([]) == []


def test_prefix_evict_forgets_both_directions():
    pc = PrefixCache(2)
    pc.record(4, [7, 8], 0)
    assert pc.has_page(4) and pc.lookup([7, 8]) == [4]
    pc.evict(4)
    assert not pc.has_page(4) and pc.lookup([7, 8]) == []
    pc.evict(4)                                         # evicting twice is harmless


def test_prefix_rerecording_a_page_drops_its_old_content():
    pc = PrefixCache(2)
    pc.record(0, [1, 2], 0)
    pc.record(0, [3, 4], 0)
    assert pc.lookup([1, 2]) == [] and pc.lookup([3, 4]) == [0]


def test_prefix_same_content_recorded_on_a_second_page_wins_and_survives_the_first_ones_eviction():
    pc = PrefixCache(2)
    pc.record(0, [1, 2], 0)
    pc.record(1, [1, 2], 0)
    assert pc.lookup([1, 2]) == [1]
    pc.evict(0)                                         # must not take page 1's entry with it
    assert pc.lookup([1, 2]) == [1]


# ---- page pool --------------------------------------------------------------------------------
def test_pool_free_parks_recorded_pages_and_releases_the_rest():
    pool = PagePool(Allocator(2), PrefixCache(2))
    p, q = pool.alloc(), pool.alloc()
    pool.record(p, [1, 2], 0)
    pool.free(p)
    pool.free(q)
    assert pool.allocator.free_pages() == 2 and pool.lookup([1, 2]) == [p]
    assert pool.alloc() == q                             # the plain free page goes first
    assert pool.alloc() == p and pool.lookup([1, 2]) == []   # eviction told the prefix index


def test_pool_lookup_refreshes_the_lru_position():
    pool = PagePool(Allocator(2), PrefixCache(1))
    p, q = pool.alloc(), pool.alloc()
    pool.record(p, [1], 0)
    pool.record(q, [2], 0)
    pool.free(p)
    pool.free(q)
    assert pool.lookup([1]) == [p]                       # p becomes the most recently used
    assert pool.alloc() == q and pool.lookup([1]) == [p]


# ---- task table -------------------------------------------------------------------------------
def test_task_table_set_get_pop():
    t = TaskTable(4)
    t.set("a", [3, 1], 4)
    assert t.get("a") == [3, 1] and t.get_cached("a") == 4
    assert t.get("missing") == [] and t.get_cached("missing") == 0
    assert t.pop("a") == ([3, 1], 4) and t.pop("a") == ([], 0)


def test_task_table_get_ref_is_the_live_list():
    t = TaskTable(4)
    pages = t.get_ref("a")
    pages.append(9)
    assert t.get("a") == [9]


def test_table_tensor_pads_with_minus_one():
    t = TaskTable(4)
    t.set("a", [3, 1, 7], 0)
    t.set("b", [2], 0)
    tt = t.table_tensor(["b", "a", "unknown"], "cpu")
    assert tt.dtype == torch.long and tt.tolist() == [[2, -1, -1], [3, 1, 7], [-1, -1, -1]]
    assert t.table_tensor(["a"], "cpu", dtype=torch.int32).dtype == torch.int32


def test_table_tensor_of_nothing_is_empty():
    t = TaskTable(4)
    assert t.table_tensor([], "cpu").shape == (0, 0)
    assert t.table_tensor(["x"], "cpu").shape == (1, 0)


# ---- K/V storage ------------------------------------------------------------------------------
def _storage(pages=6, page_size=4):
    return Storage(2, pages, page_size, 2, 8, "cpu", torch.float32)


def test_storage_write_and_gather_inside_one_page():
    st = _storage()
    table = torch.tensor([[2]])
    k, v = torch.randn(1, 3, 2, 8), torch.randn(1, 3, 2, 8)
    st.write(0, table, 0, k, v)
    gk, gv = st.gather(0, table, 3)
    assert torch.equal(gk, k) and torch.equal(gv, v)
    assert torch.equal(st.k_cache[0, 2, :3], k[0]) and (st.k_cache[1] == 0).all()      # the other layer is untouched


def test_storage_write_crosses_page_boundaries():
    st = _storage()
    table = torch.tensor([[5, 0, 3]])
    k, v = torch.randn(1, 10, 2, 8), torch.randn(1, 10, 2, 8)
    st.write(1, table, 0, k, v)
    assert torch.equal(st.k_cache[1, 5], k[0, :4]) and torch.equal(st.k_cache[1, 0], k[0, 4:8])
    assert torch.equal(st.v_cache[1, 3, :2], v[0, 8:])
    gk, _ = st.gather(1, table, 10)
    assert torch.equal(gk, k)


def test_storage_appends_at_a_start_position():
    st = _storage()
    table = torch.tensor([[1, 4]])
    first, second = torch.randn(1, 3, 2, 8), torch.randn(1, 2, 2, 8)
    st.write(0, table, 0, first, first)
    st.write(0, table, 3, second, second)                # positions 3 and 4: end of page 1, start of page 4
    gk, _ = st.gather(0, table, 5)
    assert torch.equal(gk[0, :3], first[0]) and torch.equal(gk[0, 3:], second[0])


def test_storage_gather_cuts_to_the_requested_length():
    st = _storage()
    table = torch.tensor([[0, 1]])
    k = torch.randn(1, 8, 2, 8)
    st.write(0, table, 0, k, k)
    assert st.gather(0, table, 5)[0].shape == (1, 5, 2, 8)
    assert torch.equal(st.gather(0, table, 5)[0], k[:, :5])


def test_storage_rows_of_missing_pages_read_as_zero_and_are_not_written():
    st = _storage()
    table = torch.tensor([[0, 2], [1, -1]])
    k = torch.randn(2, 8, 2, 8)
    st.write(0, table, 0, k, k)
    gk, gv = st.gather(0, table, 8)
    assert torch.equal(gk[0], k[0]) and torch.equal(gk[1, :4], k[1, :4])
    assert (gk[1, 4:] == 0).all() and (gv[1, 4:] == 0).all()
    assert (st.k_cache[0, 5] == 0).all()                 # page -1 did not alias the last page of the pool


def test_storage_slots_address_the_flat_pool():
    st = _storage(page_size=4)
    table = torch.tensor([[3, 1, -1]])
    pos = torch.tensor([[0, 3, 4, 7, 8]])
    assert st.slots(table, pos).tolist() == [[12, 15, 4, 7, -1]]


def test_storage_separate_value_width():
    st = Storage(1, 2, 4, 2, 8, "cpu", torch.float32, v_head_dim=16)
    assert st.k_cache.shape == (1, 2, 4, 2, 8) and st.v_cache.shape == (1, 2, 4, 2, 16)
    k, v = torch.randn(1, 4, 2, 8), torch.randn(1, 4, 2, 16)
    st.write(0, torch.tensor([[1]]), 0, k, v)
    gk, gv = st.gather(0, torch.tensor([[1]]), 4)
    assert torch.equal(gk, k) and torch.equal(gv, v)


# ---- per-task accounting ------------------------------------------------------------------------
def _kv(pages=4, page_size=4):
    return KVCache(1, pages, page_size, 2, 8, "cpu", torch.float32)


def test_task_alloc_takes_one_page_per_started_page_of_the_prompt():
    kv = _kv(pages=8)
    assert kv.task_alloc("a", list(range(9)))            # 9 tokens, 4 per page: 3 pages
    assert len(kv._table.get("a")) == 3 and kv.free_pages() == 5 and kv.task_cached("a") == 0
    assert kv.task_alloc("b", [1])
    assert len(kv._table.get("b")) == 1


def test_task_extend_allocates_only_when_a_new_page_starts():
    kv = _kv()
    kv.task_alloc("a", list(range(4)))                   # exactly one full page
    assert kv.task_extend("a", 3) and len(kv._table.get("a")) == 1
    assert kv.task_extend("a", 4) and len(kv._table.get("a")) == 2
    assert kv.task_extend("a", 7) and len(kv._table.get("a")) == 2
    assert kv.task_extend("a", 12) and len(kv._table.get("a")) == 4      # may jump several pages at once


def test_task_extend_reports_an_exhausted_pool():
    kv = _kv(pages=2)
    kv.task_alloc("a", list(range(8)))
    assert kv.free_pages() == 0 and not kv.task_extend("a", 8)
    kv.task_free("a")
    assert kv.free_pages() == 2


def test_failed_task_alloc_leaks_nothing():
    kv = _kv(pages=3)
    kv.task_alloc("a", list(range(8)))                   # 2 of 3 pages
    assert not kv.task_alloc("b", list(range(100, 108)))  # needs 2, one left
    assert kv.free_pages() == 1 and kv._table.get("b") == []
    assert kv.task_alloc("c", [1, 2])                    # the remaining page is still usable


def test_prompts_with_a_common_prefix_share_its_pages():
    kv = _kv(pages=6)
    prompt = list(range(10))
    kv.task_alloc("a", prompt)
    kv.task_record_hashes("a", prompt)
    other = prompt[:8] + [77, 78, 79]
    assert kv.task_alloc("b", other) and kv.task_cached("b") == 8
    assert kv._table.get("b")[:2] == kv._table.get("a")[:2] and kv._table.get("b")[2] != kv._table.get("a")[2]
    assert kv.free_pages() == 6 - 3 - 1                  # b needed one page of its own
    kv.task_free("a")
    assert kv.free_pages() == 3                           # the shared pages are still held by b
    assert kv.task_alloc("c", prompt[:8] + [5]) and kv.task_cached("c") == 8


def test_recorded_pages_survive_their_task_until_evicted():
    kv = _kv(pages=2)
    prompt = list(range(4))
    kv.task_alloc("a", prompt)
    kv.task_record_hashes("a", prompt)
    kv.task_free("a")
    assert kv.free_pages() == 2
    kv.task_alloc("b", prompt + [9])
    assert kv.task_cached("b") == 4                       # served from the parked page
    kv.task_free("b")
    kv.task_alloc("c", list(range(50, 58)))               # needs both pages: the parked one is evicted
    kv.task_free("c")
    kv.task_alloc("d", prompt + [9])
    assert kv.task_cached("d") == 0


def test_fully_cached_prompt_allocates_nothing_new():
    kv = _kv(pages=4)
    prompt = list(range(8))
    kv.task_alloc("a", prompt)
    kv.task_record_hashes("a", prompt)
    before = kv.free_pages()
    assert kv.task_alloc("b", prompt) and kv.task_cached("b") == 8 and kv.free_pages() == before


def test_table_tensor_and_view_from_the_facade():
    kv = _kv(pages=4)
    kv.task_alloc("a", list(range(6)))
    kv.task_alloc("b", [1])
    table = kv.make_table_tensor(["a", "b"], "cpu")
    assert table.shape == (2, 2) and table[1, 1] == -1
    view = kv.bind(table, total_len=6)
    k = torch.randn(2, 6, 2, 8)
    view.write(0, k, k)
    gk, _ = view.gather(0)
    assert torch.equal(gk[0], k[0]) and torch.equal(gk[1, :4], k[1, :4]) and (gk[1, 4:] == 0).all()
