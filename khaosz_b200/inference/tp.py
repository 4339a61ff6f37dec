"""Tensor-parallel serving: one process per GPU, rank 0 owns the scheduler (and the HTTP server).

The reference's engine is a single process on a single GPU (``astrai/inference/engine.py:93-116``).
Here every rank holds its slice of the weights (the same slicing as tensor-parallel training:
this rank's query heads with their KV heads, its slice of the MLP) and the KV pages of its own KV
heads; activations are replicated.  Column-parallel projections are plain local GEMMs, the
row-parallel ones (``o_proj``, ``down``) end in an all-reduce that the decode path runs as the fused
GEMM -> all-reduce kernel over NVLink (``khaosz_b200.parallel.tensor_parallel``; ``torch.distributed``
on CPU/gloo and for very long prefills).

Control flow: rank 0 runs the normal ``InferenceScheduler`` with a ``DistributedExecutor``; before
every model call it announces the call to the other ranks - a small header on a gloo control group
(so that idle workers block on the host, not in a device collective) followed by the input tensors
on the main group - and every rank then executes the same tensor-level step
(``Executor._prefill_body`` / ``_run_slot``).  Only rank 0 uses the sampled tokens; the next step's
inputs are announced again, so the workers carry no request state besides their KV pages.
"""

from __future__ import annotations

import os

import datetime
from typing import Dict, Optional

import torch
import torch.distributed as dist
import torch.nn as nn
from torch import Tensor

from .. import ops
from ..ops import attention as attn_ops
from ..parallel.tensor_parallel import _RowParallelFn
from ..parallel.tp_model import TPAttention, TPInfo, TPMLAttention, TPMLP, reject_adapters
from .core.cache import KVCache
from .core.executor import Executor

OP_STOP, OP_PREFILL, OP_DECODE, OP_SLOT = 0, 1, 2, 3
# The fused GEMM -> all-reduce kernel is a decode kernel: a handful of tiles per rank and three
# cross-rank waits.  Prefill-sized inputs take a local GEMM followed by a collective instead.
FUSED_ALLREDUCE_MAX_ROWS = int(os.environ.get("KHAOSZ_B200_TP_FUSED_AR_ROWS", "512"))


def _row_all_reduce(x: Tensor, w: Tensor, info: TPInfo) -> Tensor:
    """``all_reduce(x @ w.T)`` over the tensor-parallel group; ``x`` is ``[rows, k_local]``."""
    if info.ws == 1:
        return ops.linear(x, w)
    if x.is_cuda and x.shape[0] <= FUSED_ALLREDUCE_MAX_ROWS:
        return _RowParallelFn.apply(x, w, info.ctx(), True)   # fused GEMM -> all-reduce kernel
    y = ops.linear(x, w)
    dist.all_reduce(y, group=info.group)
    return y


def _local_linear(x: Tensor, w: Optional[Tensor], q8) -> Tensor:
    if q8 is not None:
        from ..ops.quant import linear_w8

        return linear_w8(x, q8[0], q8[1])
    return ops.linear(x, w)


def _row_linear(x2: Tensor, w: Optional[Tensor], q8, info: TPInfo) -> Tensor:
    if q8 is None:
        return _row_all_reduce(x2, w, info)
    y = _local_linear(x2, None, q8)   # int8 weights: local GEMM with in-kernel dequantisation, then the sum
    if info.ws > 1:
        dist.all_reduce(y, group=info.group)
    return y


def _quantize(param: nn.Parameter):
    from ..ops.quant import quantize_w8

    q, s = quantize_w8(param.data)
    return q, s


class _Attention(nn.Module):
    def __init__(self, attn, info: TPInfo):
        super().__init__()
        self.inner = TPAttention(attn, info)   # weight slicing shared with tensor-parallel training
        self.info = info
        self.qkv8 = self.o8 = self.gate8 = None

    def quantize(self) -> None:
        """Weight-only int8 (per output channel of this rank's slices); the bf16 copies are dropped."""
        self.qkv8, self.o8 = _quantize(self.inner.qkv_weight), _quantize(self.inner.o_weight)
        self.inner.qkv_weight = self.inner.o_weight = None
        if self.inner.use_gate:
            self.gate8 = _quantize(self.inner.gate_weight)
            self.inner.gate_weight = None

    def forward(self, x: Tensor, rotary, paged_cache, residual: Tensor) -> Tensor:
        a = self.inner
        B, S, _ = x.shape
        hl, kl, D = a.h_local, a.kv_local, a.head_dim
        cs, pos = rotary
        qkv = _local_linear(x, a.qkv_weight, self.qkv8).view(B, S, hl + 2 * kl, D)
        if paged_cache is not None and paged_cache.fused_rope_write_ok(qkv, D):
            # RoPE, the optional QK-norm and this rank's K/V page write in one kernel
            qw, kw = (a.q_norm.weight, a.k_norm.weight) if a.use_qk_norm else (None, None)
            q, k, v = paged_cache.fused_rope_write(a.layer_id, qkv, cs, pos, hl, kl, qw, kw,
                                                   a.q_norm.eps if a.use_qk_norm else 0.0)
            ctx = paged_cache.attention(a.layer_id, q, k, v, written=True)
        else:
            qk = ops.rope(qkv[:, :, : hl + kl], cs, pos)
            q, k, v = qk[:, :, :hl], qk[:, :, hl:], qkv[:, :, hl + kl:]
            if a.use_qk_norm:
                q, k = a.q_norm(q), a.k_norm(k)
            if paged_cache is not None:
                ctx = paged_cache.attention(a.layer_id, q, k, v)
            else:
                ctx = attn_ops.attention(q, k, v, causal=True)
        ctx = ctx.reshape(B * S, hl * D)
        if a.use_gate:
            ctx = ctx * torch.sigmoid(_local_linear(x, a.gate_weight, self.gate8).view(B * S, hl * D))
        out = _row_linear(ctx, a.o_weight, self.o8, self.info)
        return out.view(B, S, -1) + residual


class _LatentAttention(nn.Module):
    """Multi-head latent attention: local query heads, the full latent projection, local KV heads."""

    def __init__(self, attn, info: TPInfo):
        super().__init__()
        self.inner = TPMLAttention(attn, info)
        self.info = info
        self.qa8 = self.kvb8 = self.o8 = self.gate8 = None

    def quantize(self) -> None:
        a = self.inner
        self.qa8, self.kvb8, self.o8 = _quantize(a.qa_weight), _quantize(a.kv_b_weight), _quantize(a.o_weight)
        a.qa_weight = a.kv_b_weight = a.o_weight = None
        if a.use_gate:
            self.gate8 = _quantize(a.gate_weight)
            a.gate_weight = None

    def forward(self, x: Tensor, rotary, paged_cache, residual: Tensor) -> Tensor:
        a = self.inner
        B, S, _ = x.shape
        hl, kl, hd, nope = a.h_local, a.kv_local, a.head_dim, a.nope
        cs, pos = rotary
        y = _local_linear(x, a.qa_weight, self.qa8)
        q = y[..., : hl * hd].reshape(B, S, hl, hd)
        kv = _local_linear(a.kv_norm(y[..., hl * hd:].contiguous()), a.kv_b_weight, self.kvb8).view(B, S, kl, 2 * hd)
        q = torch.cat([q[..., :nope], ops.rope(q[..., nope:].contiguous(), cs, pos)], dim=-1)
        k = torch.cat([kv[..., :nope], ops.rope(kv[..., nope:hd].contiguous(), cs, pos)], dim=-1)
        v = kv[..., hd:]
        if a.use_qk_norm:
            q, k = a.q_norm(q), a.k_norm(k)
        if paged_cache is not None:
            ctx = paged_cache.attention(a.layer_id, q, k, v)
        else:
            ctx = attn_ops.attention(q, k, v, causal=True)
        ctx = ctx.reshape(B * S, hl * hd)
        if a.use_gate:
            ctx = ctx * torch.sigmoid(_local_linear(x, a.gate_weight, self.gate8).view(B * S, hl * hd))
        out = _row_linear(ctx, a.o_weight, self.o8, self.info)
        return out.view(B, S, -1) + residual


class _MLP(nn.Module):
    def __init__(self, mlp, info: TPInfo):
        super().__init__()
        self.inner = TPMLP(mlp, info)
        self.info = info
        self.gu8 = self.down8 = None

    def quantize(self) -> None:
        self.gu8, self.down8 = _quantize(self.inner.gate_up_weight), _quantize(self.inner.down_weight)
        self.inner.gate_up_weight = self.inner.down_weight = None

    def forward(self, x: Tensor, residual: Tensor) -> Tensor:
        m = self.inner
        B, S, _ = x.shape
        h = ops.swiglu(_local_linear(x, m.gate_up_weight, self.gu8))
        out = _row_linear(h.reshape(B * S, -1), m.down_weight, self.down8, self.info)
        return out.view(B, S, -1) + residual


class _Block(nn.Module):
    def __init__(self, block, info: TPInfo):
        super().__init__()
        self.input_norm, self.post_attention_norm = block.input_norm, block.post_attention_norm
        latent = hasattr(block.attention, "kv_a_proj")
        self.attention = (_LatentAttention if latent else _Attention)(block.attention, info)
        # a mixture-of-experts feed-forward stays whole on every rank (activations are replicated)
        dense = hasattr(block.mlp, "gate") and hasattr(block.mlp, "up") and hasattr(block.mlp, "down")
        self.mlp = _MLP(block.mlp, info) if dense else block.mlp

    def forward(self, x: Tensor, rotary, paged_cache) -> Tensor:
        h = self.attention(self.input_norm(x), rotary, paged_cache, x)
        return self.mlp(self.post_attention_norm(h), h)


class TPInferenceLM(nn.Module):
    """Tensor-parallel decoder for serving, built from a full ``AutoRegressiveLM`` that holds the same
    weights on every rank.  Same ``forward`` contract as the dense model (full logits on every rank)."""

    def __init__(self, model, group=None, int8: bool = False):
        super().__init__()
        reject_adapters(model, "tensor-parallel serving")
        self.info = TPInfo(group)
        self.config = model.config
        self.rotary_embedding = model.rotary_embedding
        self.embed_tokens = model.embed_tokens
        self.layers = nn.ModuleList(_Block(b, self.info) for b in model.layers)
        self.norm, self.lm_head = model.norm, model.lm_head
        if int8:
            for layer in self.layers:
                layer.attention.quantize()
                if hasattr(layer.mlp, "quantize"):
                    layer.mlp.quantize()
        self.kv_heads_local = self.layers[0].attention.inner.kv_local
        self.executor_cls = DistributedExecutor
        # the decode step is recorded as a CUDA graph only when it contains no library collective
        # (the int8 row-parallel layers sum their partial results with torch.distributed) and no
        # host read-back (the expert dispatch of a mixture-of-experts layer sizes its groups on the host)
        self.graph_safe = not int8 and all(isinstance(layer.mlp, _MLP) for layer in self.layers)
        # host-side control channel (collective: every rank builds the model at the same point)
        self.control = None
        if self.info.ws > 1:
            self.control = dist.new_group(backend="gloo", timeout=datetime.timedelta(days=7))

    def forward(self, input_ids: Tensor, input_mask: Optional[Tensor] = None, paged_cache=None,
                position_ids: Optional[Tensor] = None, logits_rows: Optional[Tensor] = None) -> Dict[str, Tensor]:
        x = self.embed_tokens(input_ids)
        rotary = self.rotary_embedding(x, position_ids)
        for layer in self.layers:
            x = layer(x, rotary, paged_cache)
        hidden = self.norm(x)
        if logits_rows is not None:
            logits = self.lm_head(hidden.reshape(-1, hidden.shape[-1])[logits_rows])
        else:
            logits = self.lm_head(hidden)
        return {"logits": logits, "hidden_states": hidden}


class DistributedExecutor(Executor):
    """Rank 0: announces every model call to the workers, then runs it.  Workers: ``worker_loop``."""

    def __init__(self, model: TPInferenceLM, tokenizer, page_cache: KVCache, device, dtype,
                 max_seq_len: Optional[int] = None, cuda_graphs: bool = True):
        super().__init__(model, tokenizer, page_cache, device, dtype, max_seq_len=max_seq_len,
                         cuda_graphs=cuda_graphs and getattr(model, "graph_safe", True))
        self.info = model.info
        self.control = model.control
        self._closed = False

    # -- wire format -----------------------------------------------------------------------------
    def _header(self, values) -> None:
        if self.control is None:
            return
        h = torch.tensor(list(values) + [0] * (6 - len(values)), dtype=torch.int64)
        dist.broadcast(h, src=0, group=self.control)

    def _send(self, *tensors: Tensor) -> None:
        if self.info.ws > 1:
            for t in tensors:
                dist.broadcast(t, src=0, group=self.info.group)

    def _recv(self, shape, dtype) -> Tensor:
        t = torch.empty(shape, dtype=dtype, device=self.device)
        dist.broadcast(t, src=0, group=self.info.group)
        return t

    # -- rank 0 ------------------------------------------------------------------------------------
    def _announce_prefill(self, ids, table, start_pos, prompt_len, last=None) -> None:
        # start_pos < 0 marks a right-padded batch whose per-sequence last positions follow
        self._header([OP_PREFILL, ids.shape[0], ids.shape[1], table.shape[1], -1 if last is not None else start_pos,
                      prompt_len])
        self._send(ids, table)
        if last is not None:
            self._send(last)

    def _announce_decode(self, ids, positions, table) -> None:
        self._header([OP_DECODE, ids.shape[0], 1, table.shape[1]])
        self._send(ids, positions, table)

    def _announce_slot(self, slot, n) -> None:
        self._header([OP_SLOT, slot.bucket, n])
        self._send(slot.stage)      # ids, positions, lengths, block table and sampling parameters in one piece

    def close(self) -> None:
        if not self._closed and self.info.rank == 0:
            self._closed = True
            self._header([OP_STOP])

    # -- ranks > 0 ---------------------------------------------------------------------------------
    @torch.inference_mode()
    def worker_loop(self) -> None:
        """Execute announced steps until rank 0 closes."""
        while True:
            h = torch.zeros(6, dtype=torch.int64)
            dist.broadcast(h, src=0, group=self.control)
            op, a, b, c, d, e = h.tolist()
            if op == OP_STOP:
                return
            if op == OP_PREFILL:
                ids, table = self._recv((a, b), torch.long), self._recv((a, c), torch.long)
                last = self._recv((a,), torch.long) if d < 0 else None
                self._prefill_body(ids, table, max(d, 0), e, last)
            elif op == OP_DECODE:
                ids, pos, table = self._recv((a, 1), torch.long), self._recv((a, 1), torch.long), self._recv((a, c), torch.long)
                view = self.page_cache.bind(table, seq_lens=pos.squeeze(1) + 1)
                self.model(ids, paged_cache=view, position_ids=pos)
            elif op == OP_SLOT:
                slot = self._slot(a)
                dist.broadcast(slot.stage, src=0, group=self.info.group)
                self._run_slot(slot)
            else:
                raise RuntimeError(f"unknown control op {op}")


def serve_worker(model: TPInferenceLM, tokenizer, max_batch_size: int, max_seq_len: Optional[int] = None,
                 page_size: int = 128) -> None:
    """Entry point of ranks > 0: same KV pool geometry as rank 0's scheduler, then the worker loop."""
    config = model.config
    max_seq_len = max_seq_len or config.max_len
    first = next(model.parameters())
    n_pages = (max_batch_size * (max_seq_len + page_size) + page_size - 1) // page_size
    cache = KVCache(config.n_layers, n_pages, page_size, model.kv_heads_local, config.dim // config.n_heads,
                    first.device, first.dtype)
    DistributedExecutor(model, tokenizer, cache, first.device, first.dtype, max_seq_len=max_seq_len).worker_loop()
