"""Token sampling: temperature -> top-k -> top-p -> draw.

The strategy classes mirror ``astrai/inference/sample.py:18-190`` (scalar or per-row tensor
parameters; temperature 1, top_k 0 and top_p 1 are exact no-ops; top_p 0 keeps exactly the
most likely token).  ``sample()`` runs the whole chain as one fused kernel for CUDA bf16
logits (greedy ``top_k == 1`` is an exact argmax) and as the strategy pipeline otherwise.
"""

from __future__ import annotations

from abc import ABC, abstractmethod
from typing import List, Optional, Union

import torch
from torch import Tensor

from ..ops import _lib
from ..ops._lib import check, lib, ptr, stream

NEG_INF = -float("inf")
Param = Union[float, int, Tensor]


class BaseSamplingStrategy(ABC):
    @abstractmethod
    def apply(self, logits: Tensor, filter_value: float = NEG_INF) -> Tensor:
        """Transform ``[batch, vocab]`` logits; filtered entries get ``filter_value``."""


def _column(value: Tensor, logits: Tensor) -> Tensor:
    return value.to(logits.device, non_blocking=True).reshape(-1, 1)


class TemperatureStrategy(BaseSamplingStrategy):
    def __init__(self, temperature: Param = 1.0):
        self.temperature = temperature

    def apply(self, logits, filter_value=NEG_INF):
        t = self.temperature
        if isinstance(t, Tensor):
            t = _column(t, logits).clamp(min=1e-8)
            return logits / t if bool((t != 1.0).any()) else logits
        return logits if t == 1.0 else logits / max(t, 1e-8)


class TopKStrategy(BaseSamplingStrategy):
    """Keep each row's k largest logits (k may differ per row; 0 disables)."""

    def __init__(self, top_k: Param = 0):
        self.top_k = top_k

    def apply(self, logits, filter_value=NEG_INF):
        vocab = logits.size(-1)
        k = self.top_k
        if isinstance(k, Tensor):
            k = k.to(logits.device, non_blocking=True).long().clamp(min=0, max=vocab).reshape(-1)
            widest = int(k.max())
            if widest <= 0:
                return logits
            top = torch.topk(logits, widest, dim=-1).values
            kth = top.gather(1, (k - 1).clamp(min=0).unsqueeze(1))
            kth = torch.where(k.unsqueeze(1) > 0, kth, torch.full_like(kth, NEG_INF))
        else:
            if k <= 0:
                return logits
            kth = torch.topk(logits, min(int(k), vocab), dim=-1).values[..., -1:]
        logits[logits < kth] = filter_value
        return logits


class TopPStrategy(BaseSamplingStrategy):
    """Nucleus filter: keep the most likely tokens up to and including the one that takes the
    cumulative probability past ``top_p``."""

    def __init__(self, top_p: Param = 1.0):
        self.top_p = top_p

    @staticmethod
    def _filter(logits: Tensor, top_p, filter_value: float) -> Tensor:
        ordered, order = torch.sort(logits, descending=True, dim=-1)
        cum = torch.cumsum(torch.softmax(ordered, dim=-1), dim=-1)
        # a token goes when the tokens ranked before it already hold more than top_p
        drop_sorted = torch.zeros_like(cum, dtype=torch.bool)
        drop_sorted[..., 1:] = cum[..., :-1] > top_p
        drop = torch.zeros_like(drop_sorted).scatter_(1, order, drop_sorted)
        logits[drop] = filter_value
        return logits

    def apply(self, logits, filter_value=NEG_INF):
        p = self.top_p
        if isinstance(p, Tensor):
            p = _column(p, logits)
            return self._filter(logits, p, filter_value) if bool((p < 1.0).any()) else logits
        return self._filter(logits, p, filter_value) if p < 1.0 else logits


class SamplingPipeline(BaseSamplingStrategy):
    def __init__(self, strategies: List[BaseSamplingStrategy]):
        self.strategies = strategies

    def apply(self, logits, filter_value=NEG_INF):
        for s in self.strategies:
            logits = s.apply(logits, filter_value)
        return logits

    @torch.no_grad()
    def sample(self, logits: Tensor, filter_value: float = NEG_INF) -> Tensor:
        filtered = self.apply(logits, filter_value)
        probs = torch.softmax(filtered, dim=-1)
        broken = ~torch.isfinite(probs).all(dim=-1)
        if bool(broken.any()):
            # a row with NaN or +inf logits has no distribution to draw from: take its largest finite-or-inf
            # entry instead of failing the whole batch (``multinomial`` raises on such rows)
            safe = torch.nan_to_num(filtered[broken], nan=float("-inf"))
            probs = probs.clone()
            probs[broken] = torch.nn.functional.one_hot(safe.argmax(dim=-1), probs.shape[-1]).to(probs.dtype)
        return torch.multinomial(probs, num_samples=1).squeeze(-1)


def _per_row(value: Param, rows: int, dtype, device) -> Tensor:
    if isinstance(value, Tensor):
        return value.to(device=device, dtype=dtype).reshape(-1).expand(rows).contiguous()
    return torch.full((rows,), value, dtype=dtype, device=device)


def fused_sample(logits: Tensor, temperature: Param, top_k: Param, top_p: Param,
                 uniform: Optional[Tensor] = None) -> Tensor:
    """One kernel launch for the whole chain; ``uniform`` ([rows] in [0,1)) makes it reproducible."""
    rows, vocab = logits.shape
    dev = logits.device
    if uniform is None:
        uniform = torch.rand(rows, device=dev)
    out = torch.empty(rows, dtype=torch.long, device=dev)
    t = _per_row(temperature, rows, torch.float32, dev)
    k = _per_row(top_k, rows, torch.int32, dev)
    p = _per_row(top_p, rows, torch.float32, dev)
    z = logits if logits.stride(-1) == 1 else logits.contiguous()
    check(lib().kb_sample(ptr(z), ptr(t), ptr(k), ptr(p), ptr(uniform.float().contiguous()), ptr(out), rows, vocab,
                          z.stride(0), 0, stream()), "sample")
    return out


@torch.inference_mode()
def sample(logits: Tensor, temperature: Param = 1.0, top_k: Param = 0, top_p: Param = 1.0,
           filter_value: float = NEG_INF) -> Tensor:
    """Sampled token ids ``[batch]`` from raw logits ``[batch, vocab]``."""
    if (logits.is_cuda and logits.dtype == torch.bfloat16 and logits.dim() == 2 and logits.shape[1] * 4 <= 200 * 1024
            and _lib.has("kb_sample")):
        return fused_sample(logits, temperature, top_k, top_p)
    pipeline = SamplingPipeline([TemperatureStrategy(temperature), TopKStrategy(top_k), TopPStrategy(top_p)])
    return pipeline.sample(logits.float() if logits.dtype in (torch.bfloat16, torch.float16) else logits, filter_value)
