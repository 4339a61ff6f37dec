"""Feed-forward layers: SwiGLU MLP and a DeepSeek-style mixture of experts.

Reference behaviour: ``astrai/model/components/mlp.py:16-93`` (``down(up(x) * silu(gate(x)))``,
router softmax in fp32 -> top-k -> renormalise, shared experts averaged).  The MLP runs
gate and up as one GEMM over adjacent weights with the SwiGLU in that GEMM's epilogue, and the
down projection with the residual add in its epilogue.  The MoE dispatch is sort-based (one ``argsort``, no
per-expert ``nonzero`` round trips to the host).
"""

from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn
from torch import Tensor

from ... import ops
from ...factory import BaseFactory
from .layers import Linear


class FFNFactory(BaseFactory[nn.Module]):
    @classmethod
    def create(cls, ffn_type: str, **kwargs) -> nn.Module:
        return super().create(ffn_type, **kwargs)


@FFNFactory.register("mlp")
class MLP(nn.Module):
    def __init__(self, dim: int, dim_ffn: int):
        super().__init__()
        # gate before up: the fused SwiGLU kernel reads [gate | up] from one GEMM output
        self.gate = Linear(dim, dim_ffn)
        self.up = Linear(dim, dim_ffn)
        self.down = Linear(dim_ffn, dim)

    def forward(self, x: Tensor, residual: Optional[Tensor] = None) -> Tensor:
        if type(self.gate) is Linear and type(self.up) is Linear:
            # one kernel: gate|up GEMM with the SwiGLU in its epilogue (CUDA bf16, adjacent weights)
            return self.down(ops.linear_swiglu(x, self.gate.weight, self.up.weight), residual)
        else:
            from ...ops.quant import int8_multi_linear

            gu = int8_multi_linear(x, (self.gate, self.up))
            if gu is None:  # adapters (LoRA): keep each projection's own forward
                gu = torch.cat([self.gate(x), self.up(x)], dim=-1)
        return self.down(ops.swiglu(gu), residual)


@FFNFactory.register("moe")
class DeepSeekMoE(nn.Module):
    def __init__(self, dim: int, dim_ffn: int, n_routed_experts: int, n_shared_experts: int = 1,
                 n_activated_experts: int = 2, topk_method: str = "greedy"):
        super().__init__()
        self.dim = dim
        self.n_routed_experts = n_routed_experts
        self.n_shared_experts = n_shared_experts or 0
        self.n_activated_experts = n_activated_experts
        self.topk_method = topk_method
        self.router = Linear(dim, n_routed_experts)
        self.shared_experts = nn.ModuleList(MLP(dim, dim_ffn) for _ in range(self.n_shared_experts))
        self.routed_experts = nn.ModuleList(MLP(dim, dim_ffn) for _ in range(n_routed_experts))

    def route(self, flat: Tensor):
        probs = torch.softmax(self.router(flat).float(), dim=-1).to(flat.dtype)
        weights, experts = torch.topk(probs, self.n_activated_experts, dim=-1)
        return weights / weights.sum(dim=-1, keepdim=True), experts

    def forward(self, x: Tensor, residual: Optional[Tensor] = None) -> Tensor:
        shape = x.shape
        flat = x.reshape(-1, shape[-1])
        n_tok, k = flat.shape[0], self.n_activated_experts
        weights, experts = self.route(flat)
        # group the (token, slot) assignments by expert with one sort
        order = torch.argsort(experts.reshape(-1), stable=True)
        token_of = torch.div(order, k, rounding_mode="floor")
        counts = torch.bincount(experts.reshape(-1), minlength=self.n_routed_experts).tolist()
        gathered = flat[token_of]
        w_sorted = weights.reshape(-1)[order].unsqueeze(-1)
        pieces, start = [], 0
        for e, n in enumerate(counts):
            if n:
                pieces.append(self.routed_experts[e](gathered[start:start + n]))
                start += n
        out = torch.zeros_like(flat)
        if pieces:
            out.index_add_(0, token_of, torch.cat(pieces, dim=0) * w_sorted)
        if self.n_shared_experts:
            out = out + sum(e(flat) for e in self.shared_experts) / self.n_shared_experts
        out = out.view(shape)
        return out if residual is None else out + residual
