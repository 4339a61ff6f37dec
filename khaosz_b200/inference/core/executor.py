"""Model execution for the scheduler: prefill of new prompts and one decode step for *all*
running sequences at once.

Differences from ``astrai/inference/core/executor.py:15-94`` (documented divergences):
sequences of different lengths decode together (per-sequence positions, block tables and
lengths go to the paged decode kernel), the first generated token is sampled from the prefill
logits instead of feeding the last prompt token a second time, only the rows whose logits are
needed go through the lm_head GEMM, and sampling is one fused kernel with a single
device->host copy per step.

A decode step is launch bound (a few hundred small kernels), so on CUDA it is captured once per
batch-size bucket (powers of two) into a CUDA graph over static input buffers and replayed:
the step's token ids, positions, lengths, block tables and sampling parameters are copied into
those buffers, rows beyond the live batch carry length 0 and an empty block table.
"""

from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

from ..sample import sample
from .cache import KVCache
from .task import Task


class _DecodeSlot:
    """Static buffers (and, from the second use on, the captured graph) of one batch bucket."""

    def __init__(self, bucket: int, table_width: int, device):
        self.bucket = bucket
        self.ids = torch.zeros(bucket, 1, dtype=torch.long, device=device)
        self.pos = torch.zeros(bucket, 1, dtype=torch.long, device=device)
        self.lens = torch.zeros(bucket, dtype=torch.long, device=device)
        self.table = torch.full((bucket, table_width), -1, dtype=torch.long, device=device)
        self.temperature = torch.ones(bucket, dtype=torch.float32, device=device)
        self.top_k = torch.zeros(bucket, dtype=torch.int32, device=device)
        self.top_p = torch.ones(bucket, dtype=torch.float32, device=device)
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self.out: Optional[torch.Tensor] = None
        self.uses = 0


class Executor:
    def __init__(self, model, tokenizer, page_cache: KVCache, device, dtype, max_seq_len: Optional[int] = None,
                 cuda_graphs: bool = True):
        self.model, self.tokenizer, self.page_cache = model, tokenizer, page_cache
        self.device, self.dtype = device, dtype
        self.max_seq_len = max_seq_len
        self.cuda_graphs = bool(cuda_graphs) and max_seq_len is not None and torch.device(device).type == "cuda"
        self._slots: Dict[int, _DecodeSlot] = {}

    def _sample(self, logits: torch.Tensor, tasks: List[Task]) -> List[int]:
        temperature = torch.tensor([t.temperature for t in tasks], dtype=torch.float32, device=self.device)
        top_k = torch.tensor([t.top_k for t in tasks], dtype=torch.int32, device=self.device)
        top_p = torch.tensor([t.top_p for t in tasks], dtype=torch.float32, device=self.device)
        return sample(logits, temperature, top_k, top_p).tolist()

    # -- tensor-level bodies (what a tensor-parallel worker rank replays) ------------------------------
    def _prefill_body(self, ids: torch.Tensor, table: torch.Tensor, start_pos: int, prompt_len: int,
                      last: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Logits ``[B, vocab]`` of the last prompt position.  ``last`` (``[B]``, only with
        ``start_pos == 0``): index of each sequence's last real token when shorter prompts were
        right-padded to ``prompt_len`` - causal attention keeps the padding invisible to the real
        tokens, and padded positions beyond a sequence's pages are not written."""
        B, T = ids.shape
        positions = torch.arange(start_pos, prompt_len, device=ids.device).unsqueeze(0).expand(B, T)
        view = self.page_cache.bind(table, total_len=prompt_len)
        rows = torch.arange(B, device=ids.device) * T + (last if last is not None else T - 1)
        out = self.model(ids, paged_cache=view, position_ids=positions if start_pos else None, logits_rows=rows)
        return out["logits"].reshape(B, -1)

    def _decode_body(self, ids, positions, lens, table, temperature, top_k, top_p) -> torch.Tensor:
        view = self.page_cache.bind(table, seq_lens=lens)
        out = self.model(ids, paged_cache=view, position_ids=positions)
        return sample(out["logits"].reshape(ids.shape[0], -1), temperature, top_k, top_p)

    # -- hooks of the multi-rank executor (single process: nothing to do) ------------------------------
    def _announce_prefill(self, ids: torch.Tensor, table: torch.Tensor, start_pos: int, prompt_len: int,
                          last: Optional[torch.Tensor] = None) -> None:
        pass

    def _announce_decode(self, ids: torch.Tensor, positions: torch.Tensor, table: torch.Tensor) -> None:
        pass

    def _announce_slot(self, slot: "_DecodeSlot", n: int) -> None:
        pass

    @torch.inference_mode()
    def execute_prefill(self, tasks: List[Task], prompt_len: int, start_pos: int = 0) -> List[int]:
        """Run ``prompt[start_pos:prompt_len]`` of equally shaped tasks through the model, fill
        their pages and return the first generated token of each."""
        ids = torch.tensor([t.prompt_ids[start_pos:prompt_len] for t in tasks], dtype=torch.long, device=self.device)
        table = self.page_cache.make_table_tensor([t.task_id for t in tasks], self.device)
        self._announce_prefill(ids, table, start_pos, prompt_len)
        return self._sample(self._prefill_body(ids, table, start_pos, prompt_len), tasks)

    @torch.inference_mode()
    def execute_prefill_padded(self, tasks: List[Task]) -> List[int]:
        """Prefill prompts of different lengths (none served from the prefix cache) in one batch:
        right-padded to the longest, first generated token taken at each prompt's own last position."""
        lens = [len(t.prompt_ids) for t in tasks]
        width = max(lens)
        ids = torch.tensor([t.prompt_ids + [0] * (width - n) for t, n in zip(tasks, lens)], dtype=torch.long,
                           device=self.device)
        last = torch.tensor([n - 1 for n in lens], dtype=torch.long, device=self.device)
        table = self.page_cache.make_table_tensor([t.task_id for t in tasks], self.device)
        self._announce_prefill(ids, table, 0, width, last)
        return self._sample(self._prefill_body(ids, table, 0, width, last), tasks)

    def _slot(self, bucket: int) -> "_DecodeSlot":
        slot = self._slots.get(bucket)
        if slot is None:
            width = (self.max_seq_len + self.page_cache.page_size - 1) // self.page_cache.page_size + 1
            slot = self._slots[bucket] = _DecodeSlot(bucket, width, self.device)
        return slot

    def _run_slot(self, slot: "_DecodeSlot") -> torch.Tensor:
        """One decode step over the slot's static buffers: plain launches on first use, recorded on
        the second, replayed afterwards.  Returns the sampled tokens ``[bucket]``."""
        args = (slot.ids, slot.pos, slot.lens, slot.table, slot.temperature, slot.top_k, slot.top_p)
        slot.uses += 1
        if slot.uses == 1 or not self.cuda_graphs:
            return self._decode_body(*args)
        if slot.graph is None:
            torch.cuda.current_stream().synchronize()
            graph = torch.cuda.CUDAGraph()
            try:
                with torch.cuda.graph(graph, capture_error_mode="thread_local"):
                    slot.out = self._decode_body(*args)
            except Exception:  # an op that cannot be captured: keep decoding with plain launches
                self.cuda_graphs = False
                torch.cuda.synchronize()
                return self._decode_body(*args)
            slot.graph = graph
        slot.graph.replay()
        return slot.out

    def _decode_graphed(self, tasks: List[Task], last: List[int], pos: List[int]) -> List[int]:
        n = len(tasks)
        slot = self._slot(1 << max(0, math.ceil(math.log2(n))))
        pad = slot.bucket - n
        table = self.page_cache.make_table_tensor([t.task_id for t in tasks], "cpu")
        if table.shape[1] > slot.table.shape[1]:
            raise RuntimeError("block table wider than the decode graph's static table")
        slot.ids.copy_(torch.tensor(last + [0] * pad, dtype=torch.long).unsqueeze(1), non_blocking=True)
        slot.pos.copy_(torch.tensor(pos + [0] * pad, dtype=torch.long).unsqueeze(1), non_blocking=True)
        slot.lens.copy_(torch.tensor([p + 1 for p in pos] + [0] * pad, dtype=torch.long), non_blocking=True)
        slot.table.fill_(-1)
        slot.table[:n, : table.shape[1]].copy_(table, non_blocking=True)
        slot.temperature.copy_(torch.tensor([t.temperature for t in tasks] + [1.0] * pad, dtype=torch.float32))
        slot.top_k.copy_(torch.tensor([t.top_k for t in tasks] + [1] * pad, dtype=torch.int32))
        slot.top_p.copy_(torch.tensor([t.top_p for t in tasks] + [1.0] * pad, dtype=torch.float32))
        self._announce_slot(slot, n)
        return self._run_slot(slot)[:n].tolist()

    @torch.inference_mode()
    def execute_decode(self, tasks: List[Task]) -> List[int]:
        """One token for every task: input = its latest token at position ``next_pos - 1``."""
        last = [(t.output_ids[-1] if t.output_ids else t.prompt_ids[-1]) for t in tasks]
        pos = [t.next_pos - 1 for t in tasks]
        if self.cuda_graphs:
            return self._decode_graphed(tasks, last, pos)
        ids = torch.tensor(last, dtype=torch.long, device=self.device).unsqueeze(1)
        positions = torch.tensor(pos, dtype=torch.long, device=self.device).unsqueeze(1)
        table = self.page_cache.make_table_tensor([t.task_id for t in tasks], self.device)
        self._announce_decode(ids, positions, table)
        view = self.page_cache.bind(table, seq_lens=positions.squeeze(1) + 1)
        out = self.model(ids, paged_cache=view, position_ids=positions)
        return self._sample(out["logits"].reshape(len(tasks), -1), tasks)

    def close(self) -> None:
        """Release whatever the executor holds outside this process (worker ranks)."""
