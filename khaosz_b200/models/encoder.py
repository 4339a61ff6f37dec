"""Sentence-embedding encoder: the decoder trunk run bidirectionally, then pooled
(reference: ``astrai/model/encoder.py:18-99``; pooling ``mean | cls | last``, optional L2
normalisation; an LM checkpoint loads after dropping ``lm_head.weight``)."""

from __future__ import annotations

from typing import Any, Mapping, Optional

import torch
import torch.nn.functional as F
from torch import Tensor

from ..config.model_config import EncoderConfig
from .automodel import AutoModel
from .components.layers import Embedding, RMSNorm, RotaryEmbedding
from .transformer import build_blocks


@AutoModel.register("embedding")
class EmbeddingEncoder(AutoModel):
    def __init__(self, config: EncoderConfig):
        super().__init__(config)
        self.rotary_embedding = RotaryEmbedding(config.dim // config.n_heads, config.max_len,
                                                config.rope_theta or 10000.0, rope_scaling=config.rope_scaling)
        self.embed_tokens = Embedding(config.vocab_size, config.dim)
        self.layers = build_blocks(config)
        self.norm = RMSNorm(config.dim, config.norm_eps)
        self.pooling_type = config.pooling_type or "mean"
        self.normalize_embeddings = bool(config.normalize_embeddings)
        for m in self.modules():
            if callable(getattr(m, "reset_parameters", None)):
                m.reset_parameters()

    def load_state_dict(self, state_dict: Mapping[str, Any], strict: bool = True, assign: bool = False):
        sd = {k: v for k, v in state_dict.items() if k != "lm_head.weight"}
        return super().load_state_dict(sd, strict=strict, assign=assign)

    def _mask(self, x: Tensor, input_mask: Optional[Tensor]) -> Optional[Tensor]:
        if input_mask is None:
            return None
        B, S = x.shape[:2]
        keep = input_mask.to(device=x.device, dtype=torch.bool).view(B, 1, 1, S)
        neg = -torch.finfo(x.dtype).max / 2
        return torch.zeros(B, 1, S, S, dtype=x.dtype, device=x.device).masked_fill_(~keep.expand(B, 1, S, S), neg)

    def pool(self, hidden: Tensor, input_mask: Optional[Tensor]) -> Tensor:
        B = hidden.shape[0]
        if self.pooling_type == "cls":
            return hidden[:, 0]
        if self.pooling_type == "last":
            if input_mask is None:
                return hidden[:, -1]
            last = input_mask.long().sum(dim=1) - 1
            return hidden[torch.arange(B, device=hidden.device), last]
        if input_mask is None:
            return hidden.mean(dim=1)
        w = input_mask.unsqueeze(-1).to(hidden.dtype)
        return (hidden * w).sum(dim=1) / w.sum(dim=1).clamp(min=1.0)

    def forward(self, input_ids: Tensor, input_mask: Optional[Tensor] = None,
                position_ids: Optional[Tensor] = None) -> Tensor:
        assert input_ids.dim() == 2
        x = self.embed_tokens(input_ids)
        rotary = self.rotary_embedding(x, position_ids)
        mask = self._mask(x, input_mask)
        for layer in self.layers:
            x = layer(x, rotary, mask, None, causal=False)
        pooled = self.pool(self.norm(x), input_mask)
        return F.normalize(pooled, p=2, dim=-1) if self.normalize_embeddings else pooled
