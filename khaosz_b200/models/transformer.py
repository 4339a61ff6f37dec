"""Decoder-only language model.

Capability parity with ``astrai/model/transformer.py:17-152``: embed -> N pre-norm blocks ->
RMSNorm -> lm_head, returning ``{"logits", "hidden_states"}``; optional weight tying with the
reference's state-dict behaviour (tied ``lm_head.weight`` is not saved; an untied model
loading a tied checkpoint copies the embedding).
"""

from __future__ import annotations

from typing import Any, Dict, Mapping, Optional

import torch
import torch.nn as nn
from torch import Tensor

from ..config.model_config import AutoRegressiveLMConfig
from .automodel import AutoModel
from .components.block import DecoderBlock
from .components.layers import Embedding, Linear, RMSNorm, RotaryEmbedding


def process_attention_mask(input_tensor: Tensor, position_ids: Optional[Tensor], input_mask: Optional[Tensor] = None,
                           is_causal: bool = False) -> Optional[Tensor]:
    """Additive ``[B,1,S,T]`` mask from a padding mask and explicit positions.

    Like the reference, no mask is produced when ``position_ids`` is None (training and
    evaluation forwards are plain causal; padding only enters through the loss mask).
    ``T`` is taken from the mask width when one is given, so no device->host sync is needed.
    """
    if position_ids is None:
        return None
    if input_mask is not None and input_mask.dim() > 2:
        return input_mask
    B, S = input_tensor.shape[:2]
    device, dtype = input_tensor.device, input_tensor.dtype
    if input_mask is None:
        if is_causal and S > 1 and bool((position_ids[:, 0] == 0).all()):
            return None
        T = int(position_ids.max()) + 1
        keep = torch.ones(B, 1, T, dtype=torch.bool, device=device)
    else:
        T = input_mask.shape[1]
        keep = input_mask.to(device=device, dtype=torch.bool).view(B, 1, T)
    keep = keep.expand(B, S, T)
    if is_causal:
        keep = keep & (position_ids.unsqueeze(-1) >= torch.arange(T, device=device))
    neg = -torch.finfo(dtype).max / 2
    return torch.zeros(B, 1, S, T, dtype=dtype, device=device).masked_fill_(~keep.unsqueeze(1), neg)


def _block_kwargs(cfg) -> Dict[str, Any]:
    extra = {}
    if getattr(cfg, "attn_type", "gqa") == "mla":
        extra.update(kv_lora_rank=cfg.kv_lora_rank, qk_nope_head_dim=cfg.qk_nope_head_dim,
                     qk_rope_head_dim=cfg.qk_rope_head_dim)
    if getattr(cfg, "ffn_type", "mlp") == "moe":
        extra.update(n_routed_experts=cfg.n_routed_experts, n_shared_experts=cfg.n_shared_experts,
                     n_activated_experts=cfg.n_activated_experts, topk_method=cfg.topk_method)
    return extra


def build_blocks(cfg) -> nn.ModuleList:
    extra = _block_kwargs(cfg)
    return nn.ModuleList(
        DecoderBlock(cfg.dim, cfg.n_heads, cfg.dim_ffn, cfg.n_kv_heads, cfg.norm_eps, cfg.use_qk_norm,
                     cfg.use_gated_attention, i, attn_type=getattr(cfg, "attn_type", "gqa"),
                     ffn_type=getattr(cfg, "ffn_type", "mlp"), **extra)
        for i in range(cfg.n_layers))


@AutoModel.register("autoregressive_lm")
class AutoRegressiveLM(AutoModel):
    def __init__(self, config: AutoRegressiveLMConfig):
        super().__init__(config)
        rope_dim = config.qk_rope_head_dim if config.attn_type == "mla" else config.dim // config.n_heads
        self.rotary_embedding = RotaryEmbedding(rope_dim, config.max_len, config.rope_theta or 10000.0,
                                                rope_scaling=config.rope_scaling)
        self.embed_tokens = Embedding(config.vocab_size, config.dim)
        self.layers = build_blocks(config)
        self.norm = RMSNorm(config.dim, config.norm_eps)
        self.lm_head = Linear(config.dim, config.vocab_size)
        if config.tie_weight:
            self.lm_head.weight = self.embed_tokens.weight
        self.apply(self._init_weights)

    @staticmethod
    def _init_weights(module: nn.Module) -> None:
        reset = getattr(module, "reset_parameters", None)
        if callable(reset):
            reset()

    # -- checkpoint semantics of tied weights ---------------------------------------------
    def state_dict(self, *args, **kwargs):
        sd = super().state_dict(*args, **kwargs)
        if self.config.tie_weight:
            prefix = kwargs.get("prefix", "")
            sd.pop(f"{prefix}lm_head.weight", None)
        return sd

    def load_state_dict(self, state_dict: Mapping[str, Any], strict: bool = True, assign: bool = False):
        sd = dict(state_dict)
        if "lm_head.weight" not in sd and "embed_tokens.weight" in sd:
            sd["lm_head.weight"] = sd["embed_tokens.weight"]
        return super().load_state_dict(sd, strict=strict, assign=assign)

    # -- forward ----------------------------------------------------------------------------
    def forward(self, input_ids: Tensor, input_mask: Optional[Tensor] = None, paged_cache=None,
                position_ids: Optional[Tensor] = None, logits_rows: Optional[Tensor] = None) -> Dict[str, Tensor]:
        """``logits_rows`` (inference): indices into the flattened ``[B*S]`` token axis whose
        logits are wanted; the lm_head GEMM then runs on those rows only."""
        assert input_ids.dim() == 2, "input_ids must be [batch, seq]"
        x = self.embed_tokens(input_ids)
        rotary = self.rotary_embedding(x, position_ids)
        mask = None
        if paged_cache is None:
            mask = process_attention_mask(x, position_ids, input_mask, is_causal=True)
        for layer in self.layers:
            x = layer(x, rotary, mask, paged_cache)
        hidden = self.norm(x)
        if logits_rows is not None:
            logits = self.lm_head(hidden.reshape(-1, hidden.shape[-1])[logits_rows])
        else:
            logits = self.lm_head(hidden)
        return {"logits": logits, "hidden_states": hidden}

    def pack_parameters(self, with_grad: bool = False):
        """Lay all parameters out in one flat buffer (q/k/v and gate/up become adjacent so
        they run as single GEMMs).  Returns the ``FlatParameters`` handle."""
        from ..utils.flat_params import FlatParameters

        return FlatParameters(self, with_grad=with_grad)
