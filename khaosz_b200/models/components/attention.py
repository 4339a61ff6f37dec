"""Attention layers: grouped-query attention and multi-head latent attention.

Behaviour follows the reference (``astrai/model/components/attention.py:32-212``): bias-free
projections named ``q_proj/k_proj/v_proj/o_proj`` (+ ``gate``, ``q_norm``, ``k_norm``), RoPE on
interleaved pairs, QK-RMSNorm applied *after* RoPE, optional sigmoid output gate.

What differs by design: on CUDA bf16 the q/k/v projections run as one tcgen05 GEMM over the
packed weights, RoPE is applied in place on the packed projection buffer, attention runs in
the ``[B,S,H,D]`` layout with GQA handled inside the kernel (no ``repeat_kv``, no permutes),
and the residual add is the o_proj GEMM's epilogue.  For inference the layer hands q/k/v to
the ``paged_cache`` view, which writes the new K/V into the page pool and attends through
block tables instead of gathering a dense copy.
"""

from __future__ import annotations

from typing import Optional, Tuple

import torch
import torch.nn as nn
from torch import Tensor

from ... import ops
from ...factory import BaseFactory
from ...ops import attention as attn_ops
from .layers import Linear, RMSNorm

Rotary = Tuple[Tensor, Optional[Tensor]]


class AttnFactory(BaseFactory[nn.Module]):
    @classmethod
    def create(cls, attn_type: str, **kwargs) -> nn.Module:
        return super().create(attn_type, **kwargs)


def _finish(self, x: Tensor, ctx: Tensor, residual: Optional[Tensor]) -> Tensor:
    if self.use_gated_attention:
        ctx = ctx * torch.sigmoid(self.gate(x))
    return self.o_proj(ctx, residual)


@AttnFactory.register("gqa")
class GQA(nn.Module):
    def __init__(self, dim: int, n_heads: int, n_kv_heads: int, use_qk_norm: bool, norm_eps: float,
                 use_gated_attention: bool, layer_id: int):
        super().__init__()
        if dim % n_heads or n_heads % n_kv_heads:
            raise ValueError("dim must divide by n_heads and n_heads by n_kv_heads")
        self.dim, self.n_heads, self.n_kv_heads = dim, n_heads, n_kv_heads
        self.head_dim = dim // n_heads
        self.n_rep = n_heads // n_kv_heads
        self.layer_id = layer_id
        self.use_qk_norm = bool(use_qk_norm)
        self.use_gated_attention = bool(use_gated_attention)
        self.q_proj = Linear(dim, n_heads * self.head_dim)
        self.k_proj = Linear(dim, n_kv_heads * self.head_dim)
        self.v_proj = Linear(dim, n_kv_heads * self.head_dim)
        self.o_proj = Linear(dim, dim)
        if self.use_qk_norm:
            self.q_norm = RMSNorm(self.head_dim, norm_eps)
            self.k_norm = RMSNorm(self.head_dim, norm_eps)
        if self.use_gated_attention:
            self.gate = Linear(dim, dim)

    def forward(self, x: Tensor, rotary_emb: Rotary, attn_mask: Optional[Tensor] = None, paged_cache=None,
                residual: Optional[Tensor] = None, causal: bool = True) -> Tensor:
        B, S, _ = x.shape
        H, Hkv, D = self.n_heads, self.n_kv_heads, self.head_dim
        cs, pos = rotary_emb
        projs = (self.q_proj, self.k_proj, self.v_proj)
        if all(type(p) is Linear and p.bias is None for p in projs):
            qkv = ops.multi_linear(x, tuple(p.weight for p in projs))
        else:
            from ...ops.quant import int8_multi_linear

            qkv = int8_multi_linear(x, projs)   # int8 weight-only projections: one GEMM over the stacked rows
            if qkv is None:  # adapters (LoRA) or biases: keep each projection's own forward
                qkv = torch.cat([p(x) for p in projs], dim=-1)
        qkv = qkv.view(B, S, H + 2 * Hkv, D)
        if paged_cache is None and attn_mask is None and not self.use_qk_norm and attn_ops.fused_ok(qkv, D):
            ctx = attn_ops.rope_attention_packed(qkv, cs, pos, H, Hkv, causal=causal)
            return _finish(self, x, ctx.view(B, S, H * D), residual)
        if paged_cache is not None and getattr(paged_cache, "fused_rope_write_ok", lambda *_: False)(qkv, D):
            # serving: RoPE, the optional QK-norm and the K/V page write are one kernel
            qw = self.q_norm.weight if self.use_qk_norm else None
            kw = self.k_norm.weight if self.use_qk_norm else None
            eps = self.q_norm.eps if self.use_qk_norm else 0.0
            q, k, v = paged_cache.fused_rope_write(self.layer_id, qkv, cs, pos, H, Hkv, qw, kw, eps)
            ctx = paged_cache.attention(self.layer_id, q, k, v, written=True)
            return _finish(self, x, ctx.reshape(B, S, H * D), residual)
        qk = ops.rope(qkv[:, :, : H + Hkv], cs, pos)
        q, k, v = qk[:, :, :H], qk[:, :, H:], qkv[:, :, H + Hkv:]
        if self.use_qk_norm:
            q, k = self.q_norm(q), self.k_norm(k)
        if paged_cache is not None:
            ctx = paged_cache.attention(self.layer_id, q, k, v)
        else:
            ctx = attn_ops.attention(q, k, v, causal=causal and attn_mask is None, mask=attn_mask)
        return _finish(self, x, ctx.reshape(B, S, H * D), residual)


@AttnFactory.register("mla")
class MLA(nn.Module):
    """Latent-compressed K/V: ``kv_a_proj -> kv_norm -> kv_b_proj`` yields per KV head
    ``[k_nope | k_rope | v]`` with V as wide as a full head; only the rope slice is rotated."""

    def __init__(self, dim: int, n_heads: int, n_kv_heads: int, kv_lora_rank: int, qk_nope_head_dim: int,
                 qk_rope_head_dim: int, norm_eps: float, use_qk_norm: bool, use_gated_attention: bool,
                 layer_id: int):
        super().__init__()
        self.dim, self.n_heads, self.n_kv_heads = dim, n_heads, n_kv_heads
        self.kv_lora_rank = kv_lora_rank
        self.qk_nope_head_dim, self.qk_rope_head_dim = qk_nope_head_dim, qk_rope_head_dim
        self.head_dim = qk_nope_head_dim + qk_rope_head_dim
        self.n_rep = n_heads // n_kv_heads
        self.layer_id = layer_id
        self.use_qk_norm = bool(use_qk_norm)
        self.use_gated_attention = bool(use_gated_attention)
        self.q_proj = Linear(dim, n_heads * self.head_dim)
        if self.use_qk_norm:
            self.q_norm = RMSNorm(self.head_dim, norm_eps)
            self.k_norm = RMSNorm(self.head_dim, norm_eps)
        self.kv_a_proj = Linear(dim, kv_lora_rank)
        self.kv_norm = RMSNorm(kv_lora_rank, norm_eps)
        self.kv_b_proj = Linear(kv_lora_rank, n_kv_heads * 2 * self.head_dim)
        self.o_proj = Linear(dim, dim)
        if self.use_gated_attention:
            self.gate = Linear(dim, dim)

    def forward(self, x: Tensor, rotary_emb: Rotary, attn_mask: Optional[Tensor] = None, paged_cache=None,
                residual: Optional[Tensor] = None, causal: bool = True) -> Tensor:
        B, S, _ = x.shape
        cs, pos = rotary_emb
        nope, rdim, hd = self.qk_nope_head_dim, self.qk_rope_head_dim, self.head_dim
        q = self.q_proj(x).view(B, S, self.n_heads, hd)
        kv = self.kv_b_proj(self.kv_norm(self.kv_a_proj(x))).view(B, S, self.n_kv_heads, 2 * hd)
        q = torch.cat([q[..., :nope], ops.rope(q[..., nope:].contiguous(), cs, pos)], dim=-1)
        k = torch.cat([kv[..., :nope], ops.rope(kv[..., nope:hd].contiguous(), cs, pos)], dim=-1)
        v = kv[..., hd:]
        if self.use_qk_norm:
            q, k = self.q_norm(q), self.k_norm(k)
        if paged_cache is not None:
            ctx = paged_cache.attention(self.layer_id, q, k, v)
        else:
            ctx = attn_ops.attention(q, k, v, causal=causal and attn_mask is None, mask=attn_mask)
        return _finish(self, x, ctx.reshape(B, S, self.n_heads * hd), residual)
