"""Tensor-parallel (+ sequence-parallel) form of the decoder-only language model.

``tensorize(model, group)`` rewrites an ``AutoRegressiveLM`` in place-equivalent form:

* q/k/v become one column-parallel weight holding this rank's query heads and their KV heads
  (KV heads are replicated over ``ws / n_kv_heads`` ranks when there are fewer KV heads than
  ranks), gate/up one column-parallel weight, ``o_proj`` and ``down`` row-parallel weights;
* activations between those regions live as this rank's contiguous slice of the flattened
  ``[B*S]`` token axis: embedding, RMSNorm, residual adds, the final norm, the LM head and the
  loss all run on ``tokens / ws`` rows;
* the column-parallel layers run as all-gather -> GEMM and the row-parallel ones as
  GEMM -> reduce-scatter through ``khaosz_b200.parallel.tensor_parallel`` (fused NVLink
  kernels on CUDA, ``torch.distributed`` collectives on CPU/gloo).

Replicated parameters (embedding / LM head, norm weights) see different tokens on every rank,
so their gradients are summed over the group by ``reduce_replicated_grads``; the same call
sums the K/V weight gradients over the ranks that share a KV head.  ``full_state_dict``
reassembles the reference's parameter names and shapes (``astrai/model/transformer.py:60-152``)
so checkpoints stay interchangeable.

The reference ships only forward-only TP linears that no model uses
(``astrai/parallel/module.py:18-115``); this module is what wires them into training.
"""

from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import torch
import torch.distributed as dist
import torch.nn as nn
from torch import Tensor

from .. import ops
from ..ops import attention as attn_ops
from .tensor_parallel import TPContext, _ColumnParallelFn, _RowParallelFn


class TPInfo:
    def __init__(self, group=None):
        self.group = group if group is not None else dist.group.WORLD
        self.ws = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)

    def ctx(self) -> TPContext:
        return TPContext.get(self.group)


def _column(x: Tensor, w: Tensor, info: TPInfo) -> Tensor:
    if info.ws == 1:
        return ops.linear(x, w)
    return _ColumnParallelFn.apply(x, w, info.ctx())


def _row(x: Tensor, w: Tensor, info: TPInfo) -> Tensor:
    if info.ws == 1:
        return ops.linear(x, w)
    return _RowParallelFn.apply(x, w, info.ctx(), False)


def head_partition(n_heads: int, n_kv_heads: int, ws: int, rank: int) -> Tuple[int, int, int, int]:
    """``(q_heads_local, kv_heads_local, first_kv_head, kv_replicas)`` of one rank."""
    if n_heads % ws:
        raise ValueError(f"n_heads={n_heads} must divide by the tensor-parallel size {ws}")
    hl = n_heads // ws
    if n_kv_heads >= ws:
        if n_kv_heads % ws:
            raise ValueError(f"n_kv_heads={n_kv_heads} must divide by the tensor-parallel size {ws}")
        kl = n_kv_heads // ws
        return hl, kl, rank * kl, 1
    if ws % n_kv_heads:
        raise ValueError(f"tensor-parallel size {ws} must be a multiple of n_kv_heads={n_kv_heads}")
    rep = ws // n_kv_heads
    return hl, 1, rank // rep, rep


class TPAttention(nn.Module):
    """This rank's heads of a grouped-query attention layer.

    QK-RMSNorm weights act per head, so they are replicated and their gradients summed over the
    group like any replicated parameter; the sigmoid output gate (``astrai/model/components/
    attention.py:32-120``: ``ctx * sigmoid(gate(x))`` before ``o_proj``) is column-parallel with
    the rows of this rank's query heads."""

    def __init__(self, attn, info: TPInfo):
        super().__init__()
        if not hasattr(attn, "k_proj"):
            raise NotImplementedError("tensor parallelism covers grouped-query attention (not MLA)")
        self.info = info
        self.use_qk_norm = bool(getattr(attn, "use_qk_norm", False))
        self.use_gate = bool(getattr(attn, "use_gated_attention", False))
        self.layer_id = attn.layer_id
        H, Hkv, D = attn.n_heads, attn.n_kv_heads, attn.head_dim
        self.n_heads, self.n_kv_heads, self.head_dim, self.dim = H, Hkv, D, attn.dim
        hl, kl, kv0, rep = head_partition(H, Hkv, info.ws, info.rank)
        self.h_local, self.kv_local, self.kv_first, self.kv_rep = hl, kl, kv0, rep
        r = info.rank
        with torch.no_grad():
            q = attn.q_proj.weight[r * hl * D:(r + 1) * hl * D]
            k = attn.k_proj.weight[kv0 * D:(kv0 + kl) * D]
            v = attn.v_proj.weight[kv0 * D:(kv0 + kl) * D]
            self.qkv_weight = nn.Parameter(torch.cat([q, k, v], dim=0).contiguous())
            self.o_weight = nn.Parameter(attn.o_proj.weight[:, r * hl * D:(r + 1) * hl * D].contiguous())
            self.gate_weight = None
            if self.use_gate:
                self.gate_weight = nn.Parameter(attn.gate.weight[r * hl * D:(r + 1) * hl * D].contiguous())
                self.gate_weight.tp_sharded = True
        if self.use_qk_norm:
            self.q_norm, self.k_norm = attn.q_norm, attn.k_norm
        self.qkv_weight.tp_kv_rows = (hl * D, rep)   # rows from here on are shared by `rep` ranks
        self.qkv_weight.tp_sharded = True
        self.o_weight.tp_sharded = True

    def forward(self, x_shard: Tensor, rotary, batch: int, seq: int) -> Tensor:
        hl, kl, D = self.h_local, self.kv_local, self.head_dim
        cs, pos = rotary
        qkv = _column(x_shard, self.qkv_weight, self.info).view(batch, seq, hl + 2 * kl, D)
        if not self.use_qk_norm and attn_ops.fused_ok(qkv, D):
            ctx = attn_ops.rope_attention_packed(qkv, cs, pos, hl, kl, causal=True)
        else:
            qk = ops.rope(qkv[:, :, : hl + kl], cs, pos)
            q, k = qk[:, :, :hl], qk[:, :, hl:]
            if self.use_qk_norm:       # after RoPE, as in the dense layer
                q, k = self.q_norm(q), self.k_norm(k)
            ctx = attn_ops.attention(q, k, qkv[:, :, hl + kl:], causal=True)
        ctx = ctx.reshape(batch * seq, hl * D)
        if self.use_gate:
            ctx = ctx * torch.sigmoid(_column(x_shard, self.gate_weight, self.info))
        return _row(ctx, self.o_weight, self.info)


class TPMLAttention(nn.Module):
    """This rank's heads of a multi-head latent attention layer
    (``astrai/model/components/attention.py:123-212``).

    The rows of ``q_proj`` for the local heads and the whole (narrow) ``kv_a_proj`` form one
    column-parallel weight, so the latent of every token comes out of the same gathered GEMM on
    every rank; ``kv_norm`` is replicated and ``kv_b_proj`` keeps the rows of the local KV heads.
    A rank back-propagates into the latent through its own KV heads only, so the gradient of the
    ``kv_a_proj`` rows is partial per rank and is summed over the group with the replicated
    parameters' gradients."""

    def __init__(self, attn, info: TPInfo):
        super().__init__()
        self.info = info
        self.layer_id = attn.layer_id
        H, Hkv, hd = attn.n_heads, attn.n_kv_heads, attn.head_dim
        if H % info.ws or Hkv % info.ws:
            raise ValueError(f"n_heads={H} and n_kv_heads={Hkv} must divide by the tensor-parallel size {info.ws}")
        self.n_heads, self.n_kv_heads, self.head_dim = H, Hkv, hd
        self.nope, self.rank_lat = attn.qk_nope_head_dim, attn.kv_lora_rank
        hl, kl, r = H // info.ws, Hkv // info.ws, info.rank
        self.h_local, self.kv_local = hl, kl
        self.use_qk_norm = bool(getattr(attn, "use_qk_norm", False))
        self.use_gate = bool(getattr(attn, "use_gated_attention", False))
        with torch.no_grad():
            self.qa_weight = nn.Parameter(torch.cat([attn.q_proj.weight[r * hl * hd:(r + 1) * hl * hd],
                                                     attn.kv_a_proj.weight], dim=0).contiguous())
            self.kv_b_weight = nn.Parameter(attn.kv_b_proj.weight[r * kl * 2 * hd:(r + 1) * kl * 2 * hd].contiguous())
            self.o_weight = nn.Parameter(attn.o_proj.weight[:, r * hl * hd:(r + 1) * hl * hd].contiguous())
            self.gate_weight = None
            if self.use_gate:
                self.gate_weight = nn.Parameter(attn.gate.weight[r * hl * hd:(r + 1) * hl * hd].contiguous())
                self.gate_weight.tp_sharded = True
        self.kv_norm = attn.kv_norm
        if self.use_qk_norm:
            self.q_norm, self.k_norm = attn.q_norm, attn.k_norm
        self.qa_weight.tp_sharded = True
        self.qa_weight.tp_shared_rows = hl * hd     # rows from here on: the same on every rank, partial gradients
        self.kv_b_weight.tp_sharded = True
        self.o_weight.tp_sharded = True

    def forward(self, x_shard: Tensor, rotary, batch: int, seq: int) -> Tensor:
        hl, kl, hd, nope = self.h_local, self.kv_local, self.head_dim, self.nope
        cs, pos = rotary
        y = _column(x_shard, self.qa_weight, self.info)
        q = y[:, : hl * hd].reshape(batch, seq, hl, hd)
        latent = self.kv_norm(y[:, hl * hd:].contiguous())
        kv = ops.linear(latent, self.kv_b_weight).view(batch, seq, kl, 2 * hd)
        q = torch.cat([q[..., :nope], ops.rope(q[..., nope:].contiguous(), cs, pos)], dim=-1)
        k = torch.cat([kv[..., :nope], ops.rope(kv[..., nope:hd].contiguous(), cs, pos)], dim=-1)
        v = kv[..., hd:]
        if self.use_qk_norm:
            q, k = self.q_norm(q), self.k_norm(k)
        ctx = attn_ops.attention(q, k, v, causal=True).reshape(batch * seq, hl * hd)
        if self.use_gate:
            ctx = ctx * torch.sigmoid(_column(x_shard, self.gate_weight, self.info))
        return _row(ctx, self.o_weight, self.info)


class TPMLP(nn.Module):
    def __init__(self, mlp, info: TPInfo):
        super().__init__()
        if not (hasattr(mlp, "gate") and hasattr(mlp, "up") and hasattr(mlp, "down")):
            raise NotImplementedError("tensor parallelism covers the dense SwiGLU MLP (no MoE)")
        self.info = info
        f = mlp.gate.weight.shape[0]
        if f % info.ws:
            raise ValueError(f"dim_ffn={f} must divide by the tensor-parallel size {info.ws}")
        fl, r = f // info.ws, info.rank
        self.ffn, self.ffn_local = f, fl
        with torch.no_grad():
            self.gate_up_weight = nn.Parameter(
                torch.cat([mlp.gate.weight[r * fl:(r + 1) * fl], mlp.up.weight[r * fl:(r + 1) * fl]], dim=0).contiguous())
            self.down_weight = nn.Parameter(mlp.down.weight[:, r * fl:(r + 1) * fl].contiguous())
        self.gate_up_weight.tp_sharded = True
        self.down_weight.tp_sharded = True

    def forward(self, x_shard: Tensor) -> Tensor:
        gu = _column(x_shard, self.gate_up_weight, self.info)
        return _row(ops.swiglu(gu), self.down_weight, self.info)


class TPBlock(nn.Module):
    def __init__(self, block, info: TPInfo):
        super().__init__()
        self.layer_id = block.layer_id
        self.input_norm = block.input_norm
        self.post_attention_norm = block.post_attention_norm
        self.latent_attention = hasattr(block.attention, "kv_a_proj")
        self.attention = (TPMLAttention if self.latent_attention else TPAttention)(block.attention, info)
        # A mixture-of-experts feed-forward acts per token, so it runs unchanged on this rank's token
        # slice with replicated expert weights (their gradients are summed over the group like the
        # norm weights'); only the dense SwiGLU MLP is cut into column / row slices.
        self.dense_mlp = hasattr(block.mlp, "gate") and hasattr(block.mlp, "up") and hasattr(block.mlp, "down")
        self.mlp = TPMLP(block.mlp, info) if self.dense_mlp else block.mlp

    def forward(self, x: Tensor, rotary, batch: int, seq: int) -> Tensor:
        y, x = self.input_norm.fork(x)
        h = x + self.attention(y, rotary, batch, seq)
        y, h = self.post_attention_norm.fork(h)
        return h + self.mlp(y)


class _GatherTokens(torch.autograd.Function):
    """All-gather of per-token values over the group (``[n_local] -> [n_local * ws]``); the gradient
    of a rank's slice is the sum of the slices the ranks hold for it (every rank evaluates the
    same loss on the gathered values, so the copies are averaged by the executor's 1/ws)."""

    @staticmethod
    def forward(ctx, x, info):
        if x.is_cuda and torch.cuda.is_current_stream_capturing():
            # every rank reaches this point in the same micro-step, so all of them give up the
            # recording together and keep running the step with plain launches
            raise RuntimeError("a library collective cannot be part of a recorded micro-step")
        ctx.info = info
        parts = [torch.empty_like(x) for _ in range(info.ws)]
        dist.all_gather(parts, x.contiguous(), group=info.group)
        return torch.cat(parts, dim=0)

    @staticmethod
    def backward(ctx, g):
        info = ctx.info
        g = g.contiguous()
        dist.all_reduce(g, group=info.group)
        n = g.shape[0] // info.ws
        return g[info.rank * n:(info.rank + 1) * n], None


class TensorParallelLM(nn.Module):
    """Training-time tensor-parallel decoder.  ``forward`` takes the full ``[B, S]`` batch (the
    same on every rank of the group) and returns the logits of this rank's token slice as
    ``[1, B*S/ws, vocab]``; ``shard_targets`` cuts the matching slice out of a ``[B, S]`` target."""

    def __init__(self, model, group=None):
        super().__init__()
        self.info = TPInfo(group)
        self.config = model.config
        # parameter names of the dense model in optimizer order (checkpoint layout of the moments)
        self.dense_names = [n for n, _ in model.named_parameters()]
        self.rotary_embedding = model.rotary_embedding
        self.embed_tokens = model.embed_tokens
        self.layers = nn.ModuleList(TPBlock(b, self.info) for b in model.layers)
        self.norm = model.norm
        self.lm_head = model.lm_head

    # -- token slice --------------------------------------------------------------------------
    def _slice(self, n_tokens: int) -> Tuple[int, int]:
        ws = self.info.ws
        if n_tokens % ws:
            raise ValueError(f"batch*seq = {n_tokens} must divide by the tensor-parallel size {ws}")
        n = n_tokens // ws
        return self.info.rank * n, n

    def shard_targets(self, targets: Tensor) -> Tensor:
        flat = targets.reshape(-1)
        off, n = self._slice(flat.numel())
        return flat[off:off + n].unsqueeze(0)

    def gather_tokens(self, local_values: Tensor, shape) -> Tensor:
        """Per-token values of this rank's slice -> the values of all ``B*S`` tokens, reshaped to
        ``shape`` (differentiable; used for sequence-level objectives such as DPO / GRPO)."""
        flat = local_values.reshape(-1)
        if self.info.ws > 1:
            flat = _GatherTokens.apply(flat, self.info)
        return flat.view(shape)

    def loss_weight(self, local_targets: Tensor, ignore_index: int = -100,
                    full_targets: Optional[Tensor] = None) -> Tensor:
        """Factor that turns this rank's mean loss into its share of the global mean:
        ``n_local * ws / n_global`` (the executor divides by ``ws``).  Every rank of the group reads
        the same batch, so the global count comes from ``full_targets`` without a collective (and the
        step stays recordable as a CUDA graph)."""
        n_local = (local_targets != ignore_index).sum().to(torch.float32)
        if self.info.ws == 1:
            return torch.ones_like(n_local)
        if full_targets is not None:
            n_global = (full_targets != ignore_index).sum().to(torch.float32)
        else:
            if local_targets.is_cuda and torch.cuda.is_current_stream_capturing():
                return torch.ones_like(n_local)   # no library collective inside a recorded step
            n_global = n_local.clone()
            dist.all_reduce(n_global, group=self.info.group)
        return n_local * self.info.ws / n_global.clamp_min(1.0)

    def forward(self, input_ids: Tensor, input_mask: Optional[Tensor] = None, paged_cache=None,
                position_ids: Optional[Tensor] = None, logits_rows: Optional[Tensor] = None) -> Dict[str, Tensor]:
        # like the dense model, a padding mask without explicit positions does not change attention
        if paged_cache is not None or position_ids is not None or logits_rows is not None:
            raise NotImplementedError("the tensor-parallel training model runs plain causal batches only")
        B, S = input_ids.shape
        off, n = self._slice(B * S)
        x = self.embed_tokens(input_ids.reshape(-1)[off:off + n])
        rotary = self.rotary_embedding(x, None)
        for layer in self.layers:
            x = layer(x, rotary, B, S)
        hidden = self.norm(x)
        return {"logits": self.lm_head(hidden).unsqueeze(0), "hidden_states": hidden.unsqueeze(0)}

    # -- gradients of replicated / shared parameters -----------------------------------------------
    def _replicated(self) -> List[nn.Parameter]:
        seen, out = set(), []
        for p in self.parameters():
            if id(p) not in seen and not getattr(p, "tp_sharded", False) and p.requires_grad:
                seen.add(id(p))
                out.append(p)
        return out

    @torch.no_grad()
    def reduce_replicated_grads(self) -> None:
        """Sum over the group: gradients of replicated parameters (each rank saw other tokens)
        and, when KV heads are shared between ranks, the K/V rows of the packed qkv gradients.
        One coalesced all-reduce."""
        info = self.info
        if info.ws <= 1:
            return
        pieces: List[Tensor] = []
        targets: List[Tuple[Tensor, Optional[Tuple[int, int]]]] = []
        for p in self._replicated():
            if p.grad is None:     # e.g. an expert none of this rank's tokens chose: the peers may hold a gradient
                p.grad = torch.zeros_like(p)
            pieces.append(p.grad.reshape(-1))
            targets.append((p.grad, None))
        for layer in self.layers:
            att = layer.attention
            if layer.latent_attention:
                g = att.qa_weight.grad
                if g is not None:                                       # kv_a_proj rows: partial on every rank
                    shared = g[att.qa_weight.tp_shared_rows:]
                    pieces.append(shared.reshape(-1))
                    targets.append((shared, None))
                continue
            g = att.qkv_weight.grad
            if att.kv_rep > 1 and g is not None:
                row0 = att.h_local * att.head_dim
                kv = g[row0:]                                           # [2 * D, dim]
                slots = kv.new_zeros((att.n_kv_heads,) + tuple(kv.shape))
                slots[att.kv_first] = kv
                pieces.append(slots.reshape(-1))
                targets.append((kv, (att.kv_first, att.n_kv_heads)))
        if not pieces:
            return
        flat = torch.cat(pieces)
        dist.all_reduce(flat, group=info.group)
        off = 0
        for dst, slot in targets:
            if slot is None:
                n = dst.numel()
                dst.copy_(flat[off:off + n].view(dst.shape))
            else:
                first, n_slots = slot
                n = dst.numel() * n_slots
                dst.copy_(flat[off:off + n].view((n_slots,) + tuple(dst.shape))[first])
            off += n

    @torch.no_grad()
    def grad_norm_sq(self) -> Tensor:
        """Squared L2 norm of the full model's gradient (call after ``reduce_replicated_grads``):
        sharded parts are summed over the group, replicated parts counted once."""
        info = self.info
        dev = next(self.parameters()).device
        total = torch.zeros((), dtype=torch.float32, device=dev)
        seen = set()
        for p in self.parameters():
            if id(p) in seen or p.grad is None:
                continue
            seen.add(id(p))
            g = p.grad.float()
            if not getattr(p, "tp_sharded", False):
                total += g.pow(2).sum() / info.ws
            elif hasattr(p, "tp_shared_rows"):
                total += g[:p.tp_shared_rows].pow(2).sum() + g[p.tp_shared_rows:].pow(2).sum() / info.ws
            elif hasattr(p, "tp_kv_rows") and p.tp_kv_rows[1] > 1:
                row0, rep = p.tp_kv_rows
                total += g[:row0].pow(2).sum() + g[row0:].pow(2).sum() / rep
            else:
                total += g.pow(2).sum()
        if info.ws > 1:
            dist.all_reduce(total, group=info.group)
        return total

    # -- full (unsharded) state ---------------------------------------------------------------
    def _gather(self, t: Tensor) -> List[Tensor]:
        if self.info.ws == 1:
            return [t]
        parts = [torch.empty_like(t) for _ in range(self.info.ws)]
        dist.all_gather(parts, t.contiguous(), group=self.info.group)
        return parts

    @torch.no_grad()
    def full_state_dict(self, grads: bool = False) -> Dict[str, Tensor]:
        """State dict with the reference's names and full shapes, identical on every rank
        (collective).  ``grads=True`` assembles the gradients the same way (tests)."""
        return self.gather_named(lambda p: (p.grad if grads else p.data).detach())

    @torch.no_grad()
    def scatter_named(self, full: Dict[str, Tensor]) -> Dict[int, Tensor]:
        """Inverse of ``gather_named``: this rank's slices of full, dense-named tensors, keyed by
        ``id`` of the local parameter they belong to (optimizer moments from a dense checkpoint)."""
        r = self.info.rank
        out: Dict[int, Tensor] = {id(self.embed_tokens.weight): full["embed_tokens.weight"]}
        for i, layer in enumerate(self.layers):
            att, mlp = layer.attention, layer.mlp
            pre = f"layers.{i}."
            D, hl, kl = att.head_dim, att.h_local, att.kv_local
            if layer.latent_attention:
                out[id(att.qa_weight)] = torch.cat([full[pre + "attention.q_proj.weight"][r * hl * D:(r + 1) * hl * D],
                                                    full[pre + "attention.kv_a_proj.weight"]], dim=0)
                out[id(att.kv_b_weight)] = full[pre + "attention.kv_b_proj.weight"][r * kl * 2 * D:(r + 1) * kl * 2 * D]
                out[id(att.kv_norm.weight)] = full[pre + "attention.kv_norm.weight"]
            else:
                kv0 = att.kv_first
                out[id(att.qkv_weight)] = torch.cat([
                    full[pre + "attention.q_proj.weight"][r * hl * D:(r + 1) * hl * D],
                    full[pre + "attention.k_proj.weight"][kv0 * D:(kv0 + kl) * D],
                    full[pre + "attention.v_proj.weight"][kv0 * D:(kv0 + kl) * D]], dim=0)
            out[id(att.o_weight)] = full[pre + "attention.o_proj.weight"][:, r * hl * D:(r + 1) * hl * D]
            if att.use_gate:
                out[id(att.gate_weight)] = full[pre + "attention.gate.weight"][r * hl * D:(r + 1) * hl * D]
            if att.use_qk_norm:
                out[id(att.q_norm.weight)] = full[pre + "attention.q_norm.weight"]
                out[id(att.k_norm.weight)] = full[pre + "attention.k_norm.weight"]
            if layer.dense_mlp:
                fl = mlp.ffn_local
                out[id(mlp.gate_up_weight)] = torch.cat([full[pre + "mlp.gate.weight"][r * fl:(r + 1) * fl],
                                                         full[pre + "mlp.up.weight"][r * fl:(r + 1) * fl]], dim=0)
                out[id(mlp.down_weight)] = full[pre + "mlp.down.weight"][:, r * fl:(r + 1) * fl]
            else:
                for n, p in mlp.named_parameters():
                    out[id(p)] = full[pre + "mlp." + n]
            out[id(layer.input_norm.weight)] = full[pre + "input_norm.weight"]
            out[id(layer.post_attention_norm.weight)] = full[pre + "post_attention_norm.weight"]
        out[id(self.norm.weight)] = full["norm.weight"]
        if not getattr(self.config, "tie_weight", False):
            out[id(self.lm_head.weight)] = full["lm_head.weight"]
        return out

    @torch.no_grad()
    def gather_named(self, val) -> Dict[str, Tensor]:
        """``val(param)`` (a tensor shaped like the local parameter: its data, gradient, an
        optimizer moment) assembled to the dense model's names and shapes on every rank."""
        sd: Dict[str, Tensor] = {"embed_tokens.weight": val(self.embed_tokens.weight).clone()}
        for i, layer in enumerate(self.layers):
            att, mlp = layer.attention, layer.mlp
            pre = f"layers.{i}."
            D, hl, kl = att.head_dim, att.h_local, att.kv_local
            if layer.latent_attention:
                qa = val(att.qa_weight)
                sd[pre + "attention.q_proj.weight"] = torch.cat([w[: hl * D] for w in self._gather(qa[: hl * D])], dim=0)
                sd[pre + "attention.kv_a_proj.weight"] = qa[hl * D:].clone()     # the same on every rank
                sd[pre + "attention.kv_norm.weight"] = val(att.kv_norm.weight).clone()
                sd[pre + "attention.kv_b_proj.weight"] = torch.cat(self._gather(val(att.kv_b_weight)), dim=0)
            else:
                rep = att.kv_rep
                qkv = self._gather(val(att.qkv_weight))
                sd[pre + "attention.q_proj.weight"] = torch.cat([w[: hl * D] for w in qkv], dim=0)
                owners = qkv[::rep]  # one rank per KV head group
                sd[pre + "attention.k_proj.weight"] = torch.cat([w[hl * D:(hl + kl) * D] for w in owners], dim=0)
                sd[pre + "attention.v_proj.weight"] = torch.cat([w[(hl + kl) * D:] for w in owners], dim=0)
            sd[pre + "attention.o_proj.weight"] = torch.cat(self._gather(val(att.o_weight)), dim=1)
            if att.use_gate:
                sd[pre + "attention.gate.weight"] = torch.cat(self._gather(val(att.gate_weight)), dim=0)
            if att.use_qk_norm:
                sd[pre + "attention.q_norm.weight"] = val(att.q_norm.weight).clone()
                sd[pre + "attention.k_norm.weight"] = val(att.k_norm.weight).clone()
            if layer.dense_mlp:
                gu = self._gather(val(mlp.gate_up_weight))
                fl = mlp.ffn_local
                sd[pre + "mlp.gate.weight"] = torch.cat([w[:fl] for w in gu], dim=0)
                sd[pre + "mlp.up.weight"] = torch.cat([w[fl:] for w in gu], dim=0)
                sd[pre + "mlp.down.weight"] = torch.cat(self._gather(val(mlp.down_weight)), dim=1)
            else:
                for n, p in mlp.named_parameters():
                    sd[pre + "mlp." + n] = val(p).clone()
            sd[pre + "input_norm.weight"] = val(layer.input_norm.weight).clone()
            sd[pre + "post_attention_norm.weight"] = val(layer.post_attention_norm.weight).clone()
        sd["norm.weight"] = val(self.norm.weight).clone()
        if not getattr(self.config, "tie_weight", False):
            sd["lm_head.weight"] = val(self.lm_head.weight).clone()
        return sd


def reject_adapters(model, what: str) -> None:
    """The sliced / sharded layers are built from the projections' base weights; adapters wrapped
    around them would be dropped without a trace, so they are refused instead."""
    from ..models.components.lora import LoRALinear

    wrapped = [name for name, mod in model.named_modules() if isinstance(mod, LoRALinear) and not mod._merged]
    if wrapped:
        raise NotImplementedError(f"{what} does not carry LoRA adapters ({len(wrapped)} wrapped layers, e.g. "
                                  f"{wrapped[0]}): merge them first (merge_lora) or train with none / ddp / fsdp")


def tensorize(model, group=None) -> TensorParallelLM:
    """Tensor-parallel form of an ``AutoRegressiveLM`` (weights are sliced from the full model,
    which must hold the same values on every rank)."""
    if isinstance(model, TensorParallelLM):
        return model
    if not (hasattr(model, "layers") and hasattr(model, "embed_tokens") and hasattr(model, "lm_head")):
        raise NotImplementedError(f"tensor parallelism is implemented for decoder LMs, not {type(model).__name__}")
    reject_adapters(model, "tensor parallelism")
    return TensorParallelLM(model, group)
