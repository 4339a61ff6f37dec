"""Fully sharded form of the decoder-only language model (weights sharded, gathered in the GEMM).

``full_shard(model, group)`` turns every block's projection weights into row shards of the
packed matrices ``[q;k;v]``, ``o``, ``[gate;up]`` and ``down``: rank ``r`` stores rows
``[r * n / ws, (r + 1) * n / ws)`` only.  The forward and backward GEMMs gather the weight
inside the kernel (peers' shards are pulled over NVLink while the tiles of the local shard are
being computed) and the weight gradient leaves its GEMM through a reduce-scatter, so a rank
never holds a whole gradient and holds a whole weight only in one reusable image per matrix
shape (shared by all layers).  Embedding / LM head and the norm weights stay replicated; their
gradients are averaged with one coalesced all-reduce per optimizer step.

This is the behaviour of the reference's ``FULL_SHARD`` wrapper
(``astrai/parallel/executor.py:223-272``: parameters sharded, gathered for each forward and
backward, gradients reduce-scattered) without the separate all-gather and reduce-scatter
launches.
"""

from __future__ import annotations

from typing import Dict, List, Optional

import torch
import torch.distributed as dist
import torch.nn as nn
from torch import Tensor

from .. import ops
from ..ops import attention as attn_ops
from .tensor_parallel import sharded_weight_linear
from .tp_model import TPInfo, reject_adapters


def _row_shard(w: Tensor, info: TPInfo) -> nn.Parameter:
    n = w.shape[0]
    if n % info.ws:
        raise ValueError(f"{n} weight rows do not divide by {info.ws} ranks")
    per = n // info.ws
    p = nn.Parameter(w[info.rank * per:(info.rank + 1) * per].detach().clone().contiguous())
    p.fs_sharded = True
    return p


class ShardedAttention(nn.Module):
    def __init__(self, attn, info: TPInfo):
        super().__init__()
        if not hasattr(attn, "k_proj"):
            raise NotImplementedError("full sharding covers grouped-query attention (not MLA)")
        self.info = info
        self.use_qk_norm = bool(getattr(attn, "use_qk_norm", False))
        self.use_gate = bool(getattr(attn, "use_gated_attention", False))
        if self.use_qk_norm:          # per-head norm weights: replicated, like the block norms
            self.q_norm, self.k_norm = attn.q_norm, attn.k_norm
        if self.use_gate:
            self.gate_shard = _row_shard(attn.gate.weight, info)
        self.n_heads, self.n_kv_heads, self.head_dim = attn.n_heads, attn.n_kv_heads, attn.head_dim
        self.layer_id = attn.layer_id
        with torch.no_grad():
            packed = torch.cat([attn.q_proj.weight, attn.k_proj.weight, attn.v_proj.weight], dim=0)
        self.qkv_shard = _row_shard(packed, info)
        self.o_shard = _row_shard(attn.o_proj.weight, info)

    def forward(self, x: Tensor, rotary) -> Tensor:
        B, S, _ = x.shape
        H, Hkv, D = self.n_heads, self.n_kv_heads, self.head_dim
        cs, pos = rotary
        tp = self.info.ctx()
        qkv = sharded_weight_linear(x, self.qkv_shard, tp).view(B, S, H + 2 * Hkv, D)
        if not self.use_qk_norm and attn_ops.fused_ok(qkv, D):
            ctx = attn_ops.rope_attention_packed(qkv, cs, pos, H, Hkv, causal=True)
        else:
            qk = ops.rope(qkv[:, :, : H + Hkv], cs, pos)
            q, k = qk[:, :, :H], qk[:, :, H:]
            if self.use_qk_norm:       # after RoPE, as in the dense layer
                q, k = self.q_norm(q), self.k_norm(k)
            ctx = attn_ops.attention(q, k, qkv[:, :, H + Hkv:], causal=True)
        ctx = ctx.reshape(B, S, H * D)
        if self.use_gate:
            ctx = ctx * torch.sigmoid(sharded_weight_linear(x, self.gate_shard, tp))
        return sharded_weight_linear(ctx, self.o_shard, tp)


class ShardedMLAttention(nn.Module):
    """Multi-head latent attention (``astrai/model/components/attention.py:123-212``) with every
    projection stored as a row shard and gathered inside its GEMM."""

    def __init__(self, attn, info: TPInfo):
        super().__init__()
        self.info = info
        self.n_heads, self.n_kv_heads, self.head_dim = attn.n_heads, attn.n_kv_heads, attn.head_dim
        self.nope = attn.qk_nope_head_dim
        self.layer_id = attn.layer_id
        self.use_qk_norm = bool(getattr(attn, "use_qk_norm", False))
        self.use_gate = bool(getattr(attn, "use_gated_attention", False))
        self.q_shard = _row_shard(attn.q_proj.weight, info)
        self.kv_a_shard = _row_shard(attn.kv_a_proj.weight, info)
        self.kv_b_shard = _row_shard(attn.kv_b_proj.weight, info)
        self.o_shard = _row_shard(attn.o_proj.weight, info)
        self.kv_norm = attn.kv_norm
        if self.use_qk_norm:
            self.q_norm, self.k_norm = attn.q_norm, attn.k_norm
        if self.use_gate:
            self.gate_shard = _row_shard(attn.gate.weight, info)

    def forward(self, x: Tensor, rotary) -> Tensor:
        B, S, _ = x.shape
        H, Hkv, hd, nope = self.n_heads, self.n_kv_heads, self.head_dim, self.nope
        cs, pos = rotary
        tp = self.info.ctx()
        q = sharded_weight_linear(x, self.q_shard, tp).view(B, S, H, hd)
        latent = self.kv_norm(sharded_weight_linear(x, self.kv_a_shard, tp))
        kv = sharded_weight_linear(latent, self.kv_b_shard, tp).view(B, S, Hkv, 2 * hd)
        q = torch.cat([q[..., :nope], ops.rope(q[..., nope:].contiguous(), cs, pos)], dim=-1)
        k = torch.cat([kv[..., :nope], ops.rope(kv[..., nope:hd].contiguous(), cs, pos)], dim=-1)
        v = kv[..., hd:]
        if self.use_qk_norm:
            q, k = self.q_norm(q), self.k_norm(k)
        ctx = attn_ops.attention(q, k, v, causal=True).reshape(B, S, H * hd)
        if self.use_gate:
            ctx = ctx * torch.sigmoid(sharded_weight_linear(x, self.gate_shard, tp))
        return sharded_weight_linear(ctx, self.o_shard, tp)


class ShardedMLP(nn.Module):
    def __init__(self, mlp, info: TPInfo):
        super().__init__()
        if not (hasattr(mlp, "gate") and hasattr(mlp, "up") and hasattr(mlp, "down")):
            raise NotImplementedError("full sharding covers the dense SwiGLU MLP (no MoE)")
        self.info = info
        self.ffn = mlp.gate.weight.shape[0]
        with torch.no_grad():
            packed = torch.cat([mlp.gate.weight, mlp.up.weight], dim=0)
        self.gate_up_shard = _row_shard(packed, info)
        self.down_shard = _row_shard(mlp.down.weight, info)

    def forward(self, x: Tensor) -> Tensor:
        tp = self.info.ctx()
        return sharded_weight_linear(ops.swiglu(sharded_weight_linear(x, self.gate_up_shard, tp)), self.down_shard, tp)


class ShardedBlock(nn.Module):
    def __init__(self, block, info: TPInfo):
        super().__init__()
        self.layer_id = block.layer_id
        self.input_norm = block.input_norm
        self.post_attention_norm = block.post_attention_norm
        self.latent_attention = hasattr(block.attention, "kv_a_proj")
        self.attention = (ShardedMLAttention if self.latent_attention else ShardedAttention)(block.attention, info)
        # a mixture-of-experts feed-forward stays replicated (data parallel): its expert loop issues a
        # different number of GEMMs on every rank, which in-GEMM weight gathering cannot follow
        self.dense_mlp = hasattr(block.mlp, "gate") and hasattr(block.mlp, "up") and hasattr(block.mlp, "down")
        self.mlp = ShardedMLP(block.mlp, info) if self.dense_mlp else block.mlp

    def forward(self, x: Tensor, rotary) -> Tensor:
        y, x = self.input_norm.fork(x)
        h = x + self.attention(y, rotary)
        y, h = self.post_attention_norm.fork(h)
        return h + self.mlp(y)


class FullShardLM(nn.Module):
    """Data-parallel decoder whose block weights exist as row shards only."""

    def __init__(self, model, group=None):
        super().__init__()
        self.info = TPInfo(group)
        self.config = model.config
        # parameter names of the dense model in optimizer order (checkpoint layout of the moments)
        self.dense_names = [n for n, _ in model.named_parameters()]
        self.rotary_embedding = model.rotary_embedding
        self.embed_tokens = model.embed_tokens
        self.layers = nn.ModuleList(ShardedBlock(b, self.info) for b in model.layers)
        self.norm = model.norm
        self.lm_head = model.lm_head

    def forward(self, input_ids: Tensor, input_mask: Optional[Tensor] = None, paged_cache=None,
                position_ids: Optional[Tensor] = None, logits_rows: Optional[Tensor] = None) -> Dict[str, Tensor]:
        if paged_cache is not None or position_ids is not None or logits_rows is not None:
            raise NotImplementedError("the fully sharded training model runs plain causal batches only")
        x = self.embed_tokens(input_ids)
        rotary = self.rotary_embedding(x, None)
        for layer in self.layers:
            x = layer(x, rotary)
        hidden = self.norm(x)
        return {"logits": self.lm_head(hidden), "hidden_states": hidden}

    def _replicated(self) -> List[nn.Parameter]:
        seen, out = set(), []
        for p in self.parameters():
            if id(p) not in seen and not getattr(p, "fs_sharded", False) and p.requires_grad:
                seen.add(id(p))
                out.append(p)
        return out

    @torch.no_grad()
    def reduce_replicated_grads(self) -> None:
        """Sum the replicated parameters' gradients over the group (the loss carries the 1/ws)."""
        if self.info.ws <= 1:
            return
        grads = []
        for p in self._replicated():
            if p.grad is None:      # e.g. an expert none of this rank's tokens chose: the peers may hold a gradient
                p.grad = torch.zeros_like(p)
            grads.append(p.grad)
        if not grads:
            return
        flat = torch.cat([g.reshape(-1) for g in grads])
        dist.all_reduce(flat, group=self.info.group)
        off = 0
        for g in grads:
            g.copy_(flat[off:off + g.numel()].view(g.shape))
            off += g.numel()

    @torch.no_grad()
    def grad_norm_sq(self) -> Tensor:
        """Global squared gradient norm: shards summed over the group, replicated parts once."""
        dev = next(self.parameters()).device
        total = torch.zeros((), dtype=torch.float32, device=dev)
        seen = set()
        for p in self.parameters():
            if id(p) in seen or p.grad is None:
                continue
            seen.add(id(p))
            sq = p.grad.float().pow(2).sum()
            total += sq if getattr(p, "fs_sharded", False) else sq / self.info.ws
        if self.info.ws > 1:
            dist.all_reduce(total, group=self.info.group)
        return total

    def _gather_rows(self, t: Tensor) -> Tensor:
        if self.info.ws == 1:
            return t.clone()
        parts = [torch.empty_like(t) for _ in range(self.info.ws)]
        dist.all_gather(parts, t.contiguous(), group=self.info.group)
        return torch.cat(parts, dim=0)

    @torch.no_grad()
    def full_state_dict(self) -> Dict[str, Tensor]:
        """Unsharded state dict with the reference's names, identical on every rank (collective)."""
        return self.gather_named(lambda p: p.detach())

    @torch.no_grad()
    def gather_named(self, val) -> Dict[str, Tensor]:
        """``val(param)`` (shaped like the local parameter: data, gradient, optimizer moment)
        assembled to the dense model's names and shapes on every rank."""
        sd: Dict[str, Tensor] = {"embed_tokens.weight": val(self.embed_tokens.weight).clone()}
        for i, layer in enumerate(self.layers):
            att, mlp = layer.attention, layer.mlp
            pre = f"layers.{i}."
            D, H, Hkv = att.head_dim, att.n_heads, att.n_kv_heads
            if layer.latent_attention:
                sd[pre + "attention.q_proj.weight"] = self._gather_rows(val(att.q_shard))
                sd[pre + "attention.kv_a_proj.weight"] = self._gather_rows(val(att.kv_a_shard))
                sd[pre + "attention.kv_norm.weight"] = val(att.kv_norm.weight).clone()
                sd[pre + "attention.kv_b_proj.weight"] = self._gather_rows(val(att.kv_b_shard))
            else:
                qkv = self._gather_rows(val(att.qkv_shard))
                sd[pre + "attention.q_proj.weight"] = qkv[: H * D].clone()
                sd[pre + "attention.k_proj.weight"] = qkv[H * D:(H + Hkv) * D].clone()
                sd[pre + "attention.v_proj.weight"] = qkv[(H + Hkv) * D:].clone()
            sd[pre + "attention.o_proj.weight"] = self._gather_rows(val(att.o_shard))
            if att.use_gate:
                sd[pre + "attention.gate.weight"] = self._gather_rows(val(att.gate_shard))
            if att.use_qk_norm:
                sd[pre + "attention.q_norm.weight"] = val(att.q_norm.weight).clone()
                sd[pre + "attention.k_norm.weight"] = val(att.k_norm.weight).clone()
            if layer.dense_mlp:
                gu = self._gather_rows(val(mlp.gate_up_shard))
                sd[pre + "mlp.gate.weight"] = gu[: mlp.ffn].clone()
                sd[pre + "mlp.up.weight"] = gu[mlp.ffn:].clone()
                sd[pre + "mlp.down.weight"] = self._gather_rows(val(mlp.down_shard))
            else:
                for n, p in mlp.named_parameters():
                    sd[pre + "mlp." + n] = val(p).clone()
            sd[pre + "input_norm.weight"] = val(layer.input_norm.weight).clone()
            sd[pre + "post_attention_norm.weight"] = val(layer.post_attention_norm.weight).clone()
        sd["norm.weight"] = val(self.norm.weight).clone()
        if not getattr(self.config, "tie_weight", False):
            sd["lm_head.weight"] = val(self.lm_head.weight).clone()
        return sd

    @torch.no_grad()
    def scatter_named(self, full: Dict[str, Tensor]) -> Dict[int, Tensor]:
        """Inverse of ``gather_named``: this rank's row shards of full, dense-named tensors, keyed by
        ``id`` of the local parameter (optimizer moments from a dense checkpoint)."""
        r, ws = self.info.rank, self.info.ws

        def rows(t: Tensor) -> Tensor:
            per = t.shape[0] // ws
            return t[r * per:(r + 1) * per]

        out: Dict[int, Tensor] = {id(self.embed_tokens.weight): full["embed_tokens.weight"]}
        for i, layer in enumerate(self.layers):
            att, mlp = layer.attention, layer.mlp
            pre = f"layers.{i}."
            if layer.latent_attention:
                out[id(att.q_shard)] = rows(full[pre + "attention.q_proj.weight"])
                out[id(att.kv_a_shard)] = rows(full[pre + "attention.kv_a_proj.weight"])
                out[id(att.kv_b_shard)] = rows(full[pre + "attention.kv_b_proj.weight"])
                out[id(att.kv_norm.weight)] = full[pre + "attention.kv_norm.weight"]
            else:
                out[id(att.qkv_shard)] = rows(torch.cat([full[pre + "attention.q_proj.weight"],
                                                         full[pre + "attention.k_proj.weight"],
                                                         full[pre + "attention.v_proj.weight"]], dim=0))
            out[id(att.o_shard)] = rows(full[pre + "attention.o_proj.weight"])
            if att.use_gate:
                out[id(att.gate_shard)] = rows(full[pre + "attention.gate.weight"])
            if att.use_qk_norm:
                out[id(att.q_norm.weight)] = full[pre + "attention.q_norm.weight"]
                out[id(att.k_norm.weight)] = full[pre + "attention.k_norm.weight"]
            if layer.dense_mlp:
                out[id(mlp.gate_up_shard)] = rows(torch.cat([full[pre + "mlp.gate.weight"], full[pre + "mlp.up.weight"]], dim=0))
                out[id(mlp.down_shard)] = rows(full[pre + "mlp.down.weight"])
            else:
                for n, p in mlp.named_parameters():
                    out[id(p)] = full[pre + "mlp." + n]
            out[id(layer.input_norm.weight)] = full[pre + "input_norm.weight"]
            out[id(layer.post_attention_norm.weight)] = full[pre + "post_attention_norm.weight"]
        out[id(self.norm.weight)] = full["norm.weight"]
        if not getattr(self.config, "tie_weight", False):
            out[id(self.lm_head.weight)] = full["lm_head.weight"]
        return out


def full_shard(model, group=None) -> FullShardLM:
    if isinstance(model, FullShardLM):
        return model
    if not (hasattr(model, "layers") and hasattr(model, "embed_tokens") and hasattr(model, "lm_head")):
        raise NotImplementedError(f"full sharding is implemented for decoder LMs, not {type(model).__name__}")
    reject_adapters(model, "full sharding")
    return FullShardLM(model, group)
