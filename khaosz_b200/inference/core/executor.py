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
    """Static buffers (and, from the second use on, the captured graph) of one batch bucket.

    Everything a decode step reads from the host - token ids, positions, lengths, the block table
    and the sampling parameters - lives in ONE device buffer (``stage``) with a page-locked twin on
    the host: the host fills the twin with numpy writes and one asynchronous copy moves the step's
    inputs (the reference builds a handful of small tensors per step, ``astrai/inference/core/
    executor.py:59-94``).  The named tensors below are views of ``stage``."""

    def __init__(self, bucket: int, table_width: int, device):
        self.bucket, self.width = bucket, table_width
        b, w = bucket, table_width
        tail_words = (3 * b + 1) // 2                      # three 4-byte vectors, packed into 8-byte words
        self.words = 3 * b + b * w + tail_words
        self.stage = torch.zeros(self.words, dtype=torch.long, device=device)
        on_cuda = torch.device(device).type == "cuda"
        self.host = torch.zeros(self.words, dtype=torch.long, pin_memory=on_cuda)

        def views(buf):
            tail = buf[3 * b + b * w:]
            return dict(ids=buf[0:b].view(b, 1), pos=buf[b:2 * b].view(b, 1), lens=buf[2 * b:3 * b],
                        table=buf[3 * b:3 * b + b * w].view(b, w), temperature=tail.view(torch.float32)[0:b],
                        top_p=tail.view(torch.float32)[b:2 * b], top_k=tail.view(torch.int32)[2 * b:3 * b])

        for name, t in views(self.stage).items():
            setattr(self, name, t)
        self.h = {k: v.numpy() for k, v in views(self.host).items()}
        self.h["table"][:] = -1
        self.h["temperature"][:] = 1.0
        self.h["top_p"][:] = 1.0
        self.h["top_k"][:] = 1
        self.stage.copy_(self.host)
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self.out: Optional[torch.Tensor] = None
        self.uses = 0

    def fill(self, last, pos, table_cpu, temperature, top_k, top_p) -> None:
        """Write one step's inputs into the host twin and start the (single) copy to the device."""
        n, h = len(last), self.h
        h["ids"][:n, 0] = last
        h["ids"][n:, 0] = 0
        h["pos"][:n, 0] = pos
        h["pos"][n:, 0] = 0
        h["lens"][:n] = pos
        h["lens"][:n] += 1
        h["lens"][n:] = 0
        h["table"][:] = -1
        if table_cpu.numel():
            h["table"][:n, : table_cpu.shape[1]] = table_cpu.numpy()
        h["temperature"][:n] = temperature
        h["temperature"][n:] = 1.0
        h["top_k"][:n] = top_k
        h["top_k"][n:] = 1
        h["top_p"][:n] = top_p
        h["top_p"][n:] = 1.0
        self.stage.copy_(self.host, non_blocking=True)


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
        table = self.page_cache.make_table_tensor([t.task_id for t in tasks], "cpu")
        if table.shape[1] > slot.table.shape[1]:
            raise RuntimeError("block table wider than the decode graph's static table")
        # the output of the previous step was read back (tolist) before this point, so the previous
        # copy out of the host twin has completed and the twin may be rewritten
        slot.fill(last, pos, table, [t.temperature for t in tasks], [t.top_k for t in tasks], [t.top_p for t in tasks])
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
