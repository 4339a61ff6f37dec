"""Pre-norm decoder block (reference: ``astrai/model/components/decoder_block.py:43-59``).

``h = x + attn(input_norm(x)); y = h + ffn(post_attention_norm(h))`` — both residual adds are
fused into the o_proj / down GEMM epilogues on the kernel path.
"""

from __future__ import annotations

from typing import Optional

import torch.nn as nn
from torch import Tensor

from .attention import AttnFactory
from .ffn import FFNFactory
from .layers import RMSNorm


class DecoderBlock(nn.Module):
    def __init__(self, dim: int, n_heads: int, dim_ffn: int, n_kv_heads: int, norm_eps: float, use_qk_norm: bool,
                 use_gated_attention: bool, layer_id: int, attn_type: str = "gqa", ffn_type: str = "mlp", **extra):
        super().__init__()
        self.layer_id = layer_id
        self.attention = AttnFactory.create(
            attn_type, dim=dim, n_heads=n_heads, n_kv_heads=n_kv_heads, use_qk_norm=use_qk_norm, norm_eps=norm_eps,
            use_gated_attention=use_gated_attention, layer_id=layer_id, **extra)
        self.input_norm = RMSNorm(dim, norm_eps)
        self.mlp = FFNFactory.create(ffn_type, dim=dim, dim_ffn=dim_ffn, **extra)
        self.post_attention_norm = RMSNorm(dim, norm_eps)

    def forward(self, x: Tensor, rotary_emb, attention_mask: Optional[Tensor] = None, paged_cache=None,
                causal: bool = True) -> Tensor:
        y, x = self.input_norm.fork(x)
        h = self.attention(y, rotary_emb, attention_mask, paged_cache, residual=x, causal=causal)
        y, h = self.post_attention_norm.fork(h)
        return self.mlp(y, residual=h)
