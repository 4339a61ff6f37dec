"""Paged KV cache: page allocator with ref-counts and an LRU of reusable prefix pages, a
prefix index, per-task page tables, the K/V page pools and the view objects the attention
layers talk to.

Same component roles and test-pinned behaviour as ``astrai/inference/core/cache.py:9-368``
(allocator returns -1 when exhausted, free pages are preferred over cached ones, lookups stop
at the first miss and ignore a partial last page, tables pad with -1), with three deliberate
changes: the prefix hash is *chained* (a page's hash covers every token before it, so equal
pages after different prefixes never alias), pages are written by a scatter kernel from a
slot mapping instead of a Python loop over pages, and decode attention reads K/V through the
block table inside the kernel instead of gathering a dense copy per layer per step.
"""

from __future__ import annotations

import threading
from collections import OrderedDict, deque
from typing import Callable, Dict, List, Optional, Tuple

import torch
from torch import Tensor

from ...ops import _lib
from ...ops import attention as attn_ops
from ...ops._lib import check, lib, ptr, stream

_MASK64 = (1 << 64) - 1


def page_hash(token_ids: List[int], page_idx: int, page_size: int) -> int:
    """Polynomial hash of the tokens of pages ``0..page_idx`` (chained across pages)."""
    h = 0
    for tok in token_ids[: min((page_idx + 1) * page_size, len(token_ids))]:
        h = (h * 31 + tok + 1) & _MASK64
    return h


class Allocator:
    """Page ids with reference counts.  A page whose count drops to zero either returns to the
    free list or, when it holds a reusable prefix, parks in an LRU from which it can be
    evicted (``on_evict`` tells the prefix index)."""

    def __init__(self, n_pages: int):
        self._free = deque(range(n_pages))
        self._refs = [0] * n_pages
        self._lru: "OrderedDict[int, None]" = OrderedDict()
        self.on_evict: Optional[Callable[[int], None]] = None
        self._lock = threading.Lock()

    def alloc(self) -> int:
        with self._lock:
            if self._free:
                idx = self._free.popleft()
            elif self._lru:
                idx, _ = self._lru.popitem(last=False)
                if self.on_evict:
                    self.on_evict(idx)
            else:
                return -1
            self._refs[idx] = 1
            return idx

    def free(self, idx: int, keep_cached: bool = False) -> None:
        with self._lock:
            self._refs[idx] -= 1
            if self._refs[idx] == 0:
                if keep_cached:
                    self._lru[idx] = None
                else:
                    self._free.appendleft(idx)   # most recently freed first: its lines are the warmest

    def inc_ref(self, idx: int) -> None:
        with self._lock:
            self._refs[idx] += 1
            self._lru.pop(idx, None)

    def ref_count(self, idx: int) -> int:
        with self._lock:
            return self._refs[idx]

    def touch(self, idx: int) -> None:
        with self._lock:
            if idx in self._lru:
                self._lru.move_to_end(idx)

    def free_pages(self) -> int:
        with self._lock:
            return len(self._free) + len(self._lru)


class PrefixCache:
    """hash <-> physical page, for full pages of already computed prompts."""

    def __init__(self, page_size: int):
        self._page_size = page_size
        self._page_to_hash: Dict[int, int] = {}
        self._hash_to_page: Dict[int, int] = {}
        self._lock = threading.Lock()

    def evict(self, idx: int) -> None:
        with self._lock:
            h = self._page_to_hash.pop(idx, None)
            if h is not None and self._hash_to_page.get(h) == idx:
                del self._hash_to_page[h]

    def has_page(self, idx: int) -> bool:
        with self._lock:
            return idx in self._page_to_hash

    def lookup(self, token_ids: List[int]) -> List[int]:
        hits: List[int] = []
        with self._lock:
            h = 0
            for i in range(len(token_ids) // self._page_size):
                for tok in token_ids[i * self._page_size:(i + 1) * self._page_size]:
                    h = (h * 31 + tok + 1) & _MASK64
                page = self._hash_to_page.get(h)
                if page is None:
                    break
                hits.append(page)
        return hits

    def record(self, page_idx: int, token_ids: List[int], logical_page_idx: int) -> None:
        h = page_hash(token_ids, logical_page_idx, self._page_size)
        with self._lock:
            old = self._page_to_hash.pop(page_idx, None)
            if old is not None and self._hash_to_page.get(old) == page_idx:
                del self._hash_to_page[old]
            self._page_to_hash[page_idx] = h
            self._hash_to_page[h] = page_idx


class PagePool:
    def __init__(self, allocator: Allocator, prefix: PrefixCache):
        self._alloc, self._prefix = allocator, prefix
        allocator.on_evict = prefix.evict

    @property
    def allocator(self) -> Allocator:
        return self._alloc

    @property
    def prefix(self) -> PrefixCache:
        return self._prefix

    def alloc(self) -> int:
        return self._alloc.alloc()

    def free(self, idx: int) -> None:
        keep = self._prefix.has_page(idx)
        self._alloc.free(idx, keep_cached=keep)
        if not keep:
            self._prefix.evict(idx)

    def inc_ref(self, idx: int) -> None:
        self._alloc.inc_ref(idx)

    def lookup(self, token_ids: List[int]) -> List[int]:
        hits = self._prefix.lookup(token_ids)
        for p in hits:
            self._alloc.touch(p)
        return hits

    def record(self, page_idx: int, token_ids: List[int], logical_page_idx: int) -> None:
        self._prefix.record(page_idx, token_ids, logical_page_idx)


class TaskTable:
    """task id -> (physical page list, number of prompt tokens served from the prefix cache)."""

    def __init__(self, page_size: int):
        self._page_size = page_size
        self._pages: Dict[str, List[int]] = {}
        self._cached: Dict[str, int] = {}
        self._lock = threading.Lock()

    def set(self, task_id: str, page_table: List[int], cached: int) -> None:
        with self._lock:
            self._pages[task_id], self._cached[task_id] = page_table, cached

    def get(self, task_id: str) -> List[int]:
        with self._lock:
            return self._pages.get(task_id, [])

    def get_cached(self, task_id: str) -> int:
        with self._lock:
            return self._cached.get(task_id, 0)

    def pop(self, task_id: str) -> Tuple[List[int], int]:
        with self._lock:
            return self._pages.pop(task_id, []), self._cached.pop(task_id, 0)

    def get_ref(self, task_id: str) -> List[int]:
        with self._lock:
            return self._pages.setdefault(task_id, [])

    def table_tensor(self, task_ids: List[str], device, dtype=torch.long) -> Tensor:
        with self._lock:
            rows = [list(self._pages.get(t, [])) for t in task_ids]
        width = max((len(r) for r in rows), default=0)
        return torch.tensor([r + [-1] * (width - len(r)) for r in rows], dtype=dtype, device=device).reshape(
            len(rows), width)


class Storage:
    """K and V page pools ``[n_layers, n_pages, page_size, n_kv_heads, head_dim]``."""

    def __init__(self, n_layers: int, n_pages: int, page_size: int, n_kv_heads: int, head_dim: int, device, dtype,
                 v_head_dim: Optional[int] = None):
        self.page_size, self.n_pages = page_size, n_pages
        shape = (n_layers, n_pages, page_size, n_kv_heads, head_dim)
        self.k_cache = torch.zeros(shape, device=device, dtype=dtype)
        self.v_cache = torch.zeros((*shape[:-1], v_head_dim or head_dim), device=device, dtype=dtype)

    def slots(self, page_table: Tensor, positions: Tensor) -> Tensor:
        """Flat pool row of each (sequence, position): ``page * page_size + offset``; -1 where the
        page is missing.  ``positions``: ``[B, T]``."""
        page = torch.gather(page_table.long(), 1, (positions // self.page_size).clamp(max=page_table.shape[1] - 1))
        slot = page * self.page_size + positions % self.page_size
        return torch.where(page >= 0, slot, torch.full_like(slot, -1))

    def write_slots(self, layer_id: int, slots: Tensor, k: Tensor, v: Tensor) -> None:
        """Scatter token rows ``k, v [T, Hkv, D]`` to pool rows ``slots [T]``."""
        kp = self.k_cache[layer_id].view(-1, *self.k_cache.shape[-2:])
        vp = self.v_cache[layer_id].view(-1, *self.v_cache.shape[-2:])
        same_width = k.shape[-1] == v.shape[-1]
        if (k.is_cuda and k.dtype == torch.bfloat16 and same_width and k.stride(-1) == 1 and v.stride(-1) == 1
                and k.stride(-2) == k.shape[-1] and v.stride(-2) == v.shape[-1] and (k.shape[-1] * k.shape[-2]) % 8 == 0
                and k.data_ptr() % 16 == 0 and v.data_ptr() % 16 == 0 and k.stride(0) % 8 == 0 and v.stride(0) % 8 == 0):
            row = k.shape[-2] * k.shape[-1]
            check(lib().kb_paged_kv_write(ptr(k), ptr(v), ptr(kp), ptr(vp), ptr(slots), k.shape[0], row, k.stride(0),
                                          v.stride(0), stream()), "paged_kv_write")
            return
        ok = slots >= 0
        kp.index_copy_(0, slots[ok], k[ok].to(kp.dtype))
        vp.index_copy_(0, slots[ok], v[ok].to(vp.dtype))

    def write(self, layer_id: int, page_table: Tensor, start_pos: int, k: Tensor, v: Tensor) -> None:
        """Dense batch write: ``k, v [B, T, Hkv, D]`` land at positions ``start_pos..start_pos+T``."""
        B, T = k.shape[:2]
        if T == 0:
            return
        pos = torch.arange(start_pos, start_pos + T, device=k.device).unsqueeze(0).expand(B, T)
        slots = self.slots(page_table.to(k.device), pos).reshape(-1)
        self.write_slots(layer_id, slots, k.reshape(B * T, *k.shape[2:]), v.reshape(B * T, *v.shape[2:]))

    def gather(self, layer_id: int, page_table: Tensor, total_len: int) -> Tuple[Tensor, Tensor]:
        """Dense ``[B, total_len, Hkv, D]`` copies (rows of missing pages are zero)."""
        safe = page_table.clamp(min=0).long()
        k = self.k_cache[layer_id][safe].flatten(1, 2)
        v = self.v_cache[layer_id][safe].flatten(1, 2)
        missing = page_table < 0
        if bool(missing.any()):
            rows = missing.repeat_interleave(self.page_size, dim=1)[:, :, None, None]
            k, v = k.masked_fill(rows, 0.0), v.masked_fill(rows, 0.0)
        return k[:, :total_len], v[:, :total_len]


def _pick_splits(ctas_unsplit: int, longest: int, sms: int = 148) -> int:
    """Split-KV factor of the decode kernel: the CTA count should fill whole waves of the SMs
    (one CTA per SM) while every split keeps at least two 128-key tiles; each extra split costs
    a little in the merge."""
    max_tiles = max(1, (longest + 127) // 128)
    best, best_cost = 1, None
    for n in range(1, 17):
        if n > 1 and (max_tiles + n - 1) // n < 2:
            break
        ctas = ctas_unsplit * n
        waves = (ctas + sms - 1) // sms
        cost = waves * sms / ctas * (1.0 + 0.03 * (n - 1))
        if best_cost is None or cost < best_cost - 1e-9:
            best, best_cost = n, cost
    return best


class KvcacheView:
    """What a model forward sees of the cache for one batch.

    Dense mode (``total_len``): every sequence ends at ``total_len`` and contributes the same
    number of new tokens — the reference's contract, with ``write`` / ``gather``.
    Ragged mode (``seq_lens``): sequence ``b`` ends at ``seq_lens[b]``; used by the scheduler for
    decode steps (one new token each, paged decode kernel) and single-sequence prefill.
    """

    def __init__(self, storage: Storage, page_table: Tensor, total_len: int = 0, seq_lens: Optional[Tensor] = None,
                 n_splits: int = 0):
        self._storage, self._page_table, self._total_len = storage, page_table, total_len
        self._seq_lens = seq_lens
        self._table32: Optional[Tensor] = None
        self._lens32: Optional[Tensor] = None
        self._slots: Optional[Tensor] = None
        self._n_splits = n_splits
        self._scratch = None

    # -- reference-compatible pair -----------------------------------------------------------
    def write(self, layer_id: int, k: Tensor, v: Tensor) -> None:
        if self._seq_lens is None:
            self._storage.write(layer_id, self._page_table, self._total_len - k.size(1), k, v)
        else:
            self._write_ragged(layer_id, k, v)

    def gather(self, layer_id: int) -> Tuple[Tensor, Tensor]:
        total = self._total_len if self._seq_lens is None else int(self._seq_lens.max())
        return self._storage.gather(layer_id, self._page_table, total)

    # -- fused path ----------------------------------------------------------------------------
    def _token_slots(self, B: int, T: int, device) -> Tensor:
        """Pool row of each of the ``B * T`` new tokens (cached per view: the same for every layer)."""
        if self._slots is None or self._slots.numel() != B * T:
            if self._seq_lens is None:
                pos = torch.arange(self._total_len - T, self._total_len, device=device).unsqueeze(0).expand(B, T)
            else:
                pos = self._seq_lens.long().unsqueeze(1) - T + torch.arange(T, device=device).unsqueeze(0)
            self._slots = self._storage.slots(self._page_table.to(device), pos.clamp(min=0)).reshape(-1).contiguous()
        return self._slots

    def fused_rope_write_ok(self, qkv: Tensor, head_dim: int) -> bool:
        st = self._storage
        return (qkv.is_cuda and qkv.dtype == torch.bfloat16 and qkv.is_contiguous() and head_dim in (64, 128, 256)
                and st.k_cache.shape[-1] == head_dim and st.v_cache.shape[-1] == head_dim
                and not torch.is_grad_enabled() and _lib.has("kb_rope_norm_kvwrite"))

    def fused_rope_write(self, layer_id: int, qkv: Tensor, cs: Tensor, pos: Optional[Tensor], H: int, Hkv: int,
                         q_norm_w: Optional[Tensor] = None, k_norm_w: Optional[Tensor] = None, eps: float = 1e-5):
        """One kernel for what the reference does in four steps (``astrai/model/components/attention.py:86-93``):
        rotate q and k, normalise them per head when the model has QK-norm, and store this step's K / V rows
        into their pages.  ``qkv`` is the packed projection ``[B, T, H + 2 Hkv, D]`` (rotated in place);
        returns the ``q, k, v`` views to hand to :meth:`attention` with ``written=True``."""
        B, T, _, D = qkv.shape
        slots = self._token_slots(B, T, qkv.device)
        pos32 = None if pos is None else pos.to(torch.int32).expand(B, T).contiguous()
        st = self._storage
        check(lib().kb_rope_norm_kvwrite(ptr(qkv), ptr(cs), ptr(pos32), ptr(q_norm_w), ptr(k_norm_w), float(eps),
                                         ptr(slots), ptr(st.k_cache[layer_id]), ptr(st.v_cache[layer_id]), B * T, T, H,
                                         Hkv, D, qkv.stride(1), stream()), "rope_norm_kvwrite")
        return qkv[:, :, :H], qkv[:, :, H:H + Hkv], qkv[:, :, H + Hkv:]

    def _write_ragged(self, layer_id: int, k: Tensor, v: Tensor) -> None:
        B, T = k.shape[:2]
        if self._slots is None or self._slots.numel() != B * T:
            pos = self._seq_lens.long().unsqueeze(1) - T + torch.arange(T, device=k.device).unsqueeze(0)
            self._slots = self._storage.slots(self._page_table, pos.clamp(min=0)).reshape(-1).contiguous()
        self._storage.write_slots(layer_id, self._slots, k.reshape(B * T, *k.shape[2:]), v.reshape(B * T, *v.shape[2:]))

    def _decode_kernel_ok(self, q: Tensor, k: Tensor, v: Tensor) -> bool:
        H, Hkv = q.shape[2], k.shape[2]
        return (self._seq_lens is not None and q.shape[1] == 1 and q.is_cuda and q.dtype == torch.bfloat16
                and q.shape[-1] == 128 and v.shape[-1] == 128 and H % Hkv == 0
                and H // Hkv <= (32 if self._storage.page_size in (16, 32, 64, 128) else 8)
                and _lib.has("kb_paged_decode_attn"))

    def attention(self, layer_id: int, q: Tensor, k: Tensor, v: Tensor, written: bool = False) -> Tensor:
        """Append this step's K/V to the pages (unless :meth:`fused_rope_write` already did), then attend:
        ``q [B,T,H,D]`` -> ``[B,T,H,Dv]``."""
        if not written:
            self.write(layer_id, k, v)
        B, T, H, D = q.shape
        if self._decode_kernel_ok(q, k, v):
            st = self._storage
            if self._table32 is None:
                self._table32 = self._page_table.to(torch.int32).contiguous()
                self._lens32 = self._seq_lens.to(torch.int32).contiguous()
                if not self._n_splits:
                    self._n_splits = _pick_splits(B * k.shape[2], st.page_size * self._table32.shape[1])
                self._scratch = (torch.empty(B * H * self._n_splits * 128, dtype=torch.float32, device=q.device),
                                 torch.empty(B * H * self._n_splits * 2, dtype=torch.float32, device=q.device))
            q2 = q.reshape(B, H * D)
            if q2.stride(-1) != 1:
                q2 = q2.contiguous()
            out = torch.empty((B, H * D), dtype=q.dtype, device=q.device)
            if st.page_size in (16, 32, 64, 128) and _lib.has("kb_paged_decode_tc") and q2.data_ptr() % 16 == 0:
                # tensor-core kernel: K/V pages stream through TMA once for the whole query group
                check(lib().kb_paged_decode_tc(ptr(q2), ptr(st.k_cache[layer_id]), ptr(st.v_cache[layer_id]),
                                               ptr(self._table32), ptr(self._lens32), ptr(self._scratch[0]),
                                               ptr(self._scratch[1]), ptr(out), B, H, k.shape[2], D, st.page_size,
                                               self._table32.shape[1], st.n_pages, self._n_splits, q2.stride(0),
                                               out.stride(0), float(D ** -0.5), stream()), "paged_decode_tc")
                _lib.add_launches(1 if self._n_splits > 1 else 0)
                return out.view(B, 1, H, D)
            check(lib().kb_paged_decode_attn(ptr(q2), ptr(st.k_cache[layer_id]), ptr(st.v_cache[layer_id]),
                                             ptr(self._table32), ptr(self._lens32), ptr(self._scratch[0]),
                                             ptr(self._scratch[1]), ptr(out), B, H, k.shape[2], D, st.page_size,
                                             self._table32.shape[1], self._n_splits, q2.stride(0), out.stride(0),
                                             float(D ** -0.5), stream()), "paged_decode")
            _lib.add_launches(1)
            return out.view(B, 1, H, D)
        if self._seq_lens is None:
            total = self._total_len
            start = total - T
            if start == 0:
                return attn_ops.attention(q, k, v, causal=True)
            kk, vv = self._storage.gather(layer_id, self._page_table, total)
            return attn_ops.attention(q, kk, vv, causal=True)
        if T > 1:
            # ragged multi-token step: every sequence attends with its last T positions to its own cached
            # length.  One rectangular causal attention per sequence over that sequence's pages (the flash
            # kernel for bf16 on CUDA) instead of one padded batch with an explicit mask
            if getattr(self, "_lens_host", None) is None:
                self._lens_host = [int(n) for n in self._seq_lens.tolist()]     # one read per step, not per layer
            outs = []
            for b, total in enumerate(self._lens_host):
                kk, vv = self._storage.gather(layer_id, self._page_table[b:b + 1], total)
                outs.append(attn_ops.attention(q[b:b + 1], kk, vv, causal=True))
            return torch.cat(outs, dim=0)
        # single-token step where the decode kernel does not apply (CPU, fp32, unusual head sizes): one padded
        # batch with an explicit mask
        lens = self._seq_lens.long()
        total = int(lens.max())
        kk, vv = self._storage.gather(layer_id, self._page_table, total)
        keep = torch.arange(total, device=q.device).view(1, 1, total) < lens.view(B, 1, 1)
        mask = torch.zeros(B, 1, 1, total, dtype=q.dtype, device=q.device).masked_fill_(
            ~keep.unsqueeze(1), -torch.finfo(q.dtype).max / 2)
        return attn_ops.attention(q, kk, vv, causal=False, mask=mask)


class KVCache:
    """Facade used by the scheduler: page accounting per task plus view construction."""

    def __init__(self, n_layers: int, n_pages: int, page_size: int, n_kv_heads: int, head_dim: int, device, dtype,
                 v_head_dim: Optional[int] = None):
        self.page_size = page_size
        self._pool = PagePool(Allocator(n_pages), PrefixCache(page_size))
        self._table = TaskTable(page_size)
        self._storage = Storage(n_layers, n_pages, page_size, n_kv_heads, head_dim, device, dtype, v_head_dim)

    def task_alloc(self, task_id: str, prompt_ids: List[int]) -> bool:
        hits = self._pool.lookup(prompt_ids)
        for p in hits:
            self._pool.inc_ref(p)
        cached = len(hits) * self.page_size
        need = -(-(len(prompt_ids) - cached) // self.page_size) if len(prompt_ids) > cached else 0
        fresh: List[int] = []
        for _ in range(need):
            p = self._pool.alloc()
            if p < 0:
                for q in hits + fresh:
                    self._pool.free(q)
                return False
            fresh.append(p)
        self._table.set(task_id, hits + fresh, cached)
        return True

    def task_free(self, task_id: str) -> None:
        pages, _ = self._table.pop(task_id)
        for p in pages:
            self._pool.free(p)

    def task_extend(self, task_id: str, pos: int) -> bool:
        pages = self._table.get_ref(task_id)
        while len(pages) < pos // self.page_size + 1:
            p = self._pool.alloc()
            if p < 0:
                return False
            pages.append(p)
        return True

    def task_cached(self, task_id: str) -> int:
        return self._table.get_cached(task_id)

    def task_record_hashes(self, task_id: str, prompt_ids: List[int], start_logical_page: int = 0) -> None:
        pages = self._table.get(task_id)
        for i in range(start_logical_page, min(len(prompt_ids) // self.page_size, len(pages))):
            self._pool.record(pages[i], prompt_ids, i)

    def free_pages(self) -> int:
        return self._pool.allocator.free_pages()

    def make_table_tensor(self, task_ids: List[str], device, dtype=torch.long) -> Tensor:
        return self._table.table_tensor(task_ids, device, dtype)

    def bind(self, page_table: Tensor, total_len: int = 0, seq_lens: Optional[Tensor] = None,
             n_splits: int = 0) -> KvcacheView:
        """``n_splits`` fixes the split-KV factor of the decode kernel (0: chosen from the batch)."""
        return KvcacheView(self._storage, page_table, total_len, seq_lens, n_splits)
