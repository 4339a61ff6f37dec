"""Model execution for the scheduler: prefill of new prompts and one decode step for *all*
running sequences at once.

Differences from ``astrai/inference/core/executor.py:15-94`` (documented divergences):
sequences of different lengths decode together (per-sequence positions, block tables and
lengths go to the paged decode kernel), the first generated token is sampled from the prefill
logits instead of feeding the last prompt token a second time, only the rows whose logits are
needed go through the lm_head GEMM, and sampling is one fused kernel with a single
device->host copy per step.
"""

from __future__ import annotations

from typing import List, Optional

import torch

from ..sample import sample
from .cache import KVCache
from .task import Task


class Executor:
    def __init__(self, model, tokenizer, page_cache: KVCache, device, dtype):
        self.model, self.tokenizer, self.page_cache = model, tokenizer, page_cache
        self.device, self.dtype = device, dtype

    def _sample(self, logits: torch.Tensor, tasks: List[Task]) -> List[int]:
        temperature = torch.tensor([t.temperature for t in tasks], dtype=torch.float32, device=self.device)
        top_k = torch.tensor([t.top_k for t in tasks], dtype=torch.int32, device=self.device)
        top_p = torch.tensor([t.top_p for t in tasks], dtype=torch.float32, device=self.device)
        return sample(logits, temperature, top_k, top_p).tolist()

    @torch.inference_mode()
    def execute_prefill(self, tasks: List[Task], prompt_len: int, start_pos: int = 0) -> List[int]:
        """Run ``prompt[start_pos:prompt_len]`` of equally shaped tasks through the model, fill
        their pages and return the first generated token of each."""
        ids = torch.tensor([t.prompt_ids[start_pos:prompt_len] for t in tasks], dtype=torch.long, device=self.device)
        B, T = ids.shape
        table = self.page_cache.make_table_tensor([t.task_id for t in tasks], self.device)
        positions = torch.arange(start_pos, prompt_len, device=self.device).unsqueeze(0).expand(B, T)
        view = self.page_cache.bind(table, total_len=prompt_len)
        rows = torch.arange(B, device=self.device) * T + (T - 1)
        out = self.model(ids, paged_cache=view, position_ids=positions if start_pos else None, logits_rows=rows)
        return self._sample(out["logits"].reshape(B, -1), tasks)

    @torch.inference_mode()
    def execute_decode(self, tasks: List[Task]) -> List[int]:
        """One token for every task: input = its latest token at position ``next_pos - 1``."""
        last = [(t.output_ids[-1] if t.output_ids else t.prompt_ids[-1]) for t in tasks]
        pos = [t.next_pos - 1 for t in tasks]
        ids = torch.tensor(last, dtype=torch.long, device=self.device).unsqueeze(1)
        positions = torch.tensor(pos, dtype=torch.long, device=self.device).unsqueeze(1)
        table = self.page_cache.make_table_tensor([t.task_id for t in tasks], self.device)
        view = self.page_cache.bind(table, seq_lens=positions.squeeze(1) + 1)
        out = self.model(ids, paged_cache=view, position_ids=positions)
        return self._sample(out["logits"].reshape(len(tasks), -1), tasks)
