"""Leaf modules: bias-free Linear, Embedding, RMSNorm and the rotary table.

Parameter names and shapes follow the reference (``astrai/model/components/{linear,embedding,
norm,rope}.py``) so checkpoints interchange; the forward passes call ``khaosz_b200.ops`` which
runs sm_100a kernels for CUDA bf16 tensors and plain PyTorch elsewhere.
"""

from __future__ import annotations

import math
from typing import Optional, Tuple

import torch
import torch.nn as nn
from torch import Tensor

from ... import ops


class Linear(nn.Module):
    """``y = x W^T (+ b)`` with ``W: [out, in]``; kaiming-uniform(a=sqrt(5)) init."""

    def __init__(self, in_dim: int, out_dim: int, bias: bool = False):
        super().__init__()
        self.in_dim, self.out_dim = in_dim, out_dim
        self.weight = nn.Parameter(torch.empty(out_dim, in_dim))
        self.bias = nn.Parameter(torch.zeros(out_dim)) if bias else None
        self.reset_parameters()

    def reset_parameters(self) -> None:
        nn.init.kaiming_uniform_(self.weight, a=math.sqrt(5))
        if self.bias is not None:
            nn.init.zeros_(self.bias)

    def forward(self, x: Tensor, residual: Optional[Tensor] = None) -> Tensor:
        y = ops.linear(x, self.weight, residual)
        return y if self.bias is None else y + self.bias

    def extra_repr(self) -> str:
        return f"in={self.in_dim}, out={self.out_dim}, bias={self.bias is not None}"


class Embedding(nn.Module):
    """Token table ``[vocab, dim]`` initialised N(0, 0.02)."""

    def __init__(self, vocab_size: int, dim: int):
        super().__init__()
        self.weight = nn.Parameter(torch.empty(vocab_size, dim))
        self.reset_parameters()

    def reset_parameters(self) -> None:
        nn.init.normal_(self.weight, mean=0.0, std=0.02)

    def forward(self, ids: Tensor) -> Tensor:
        return ops.embedding(ids, self.weight)


class RMSNorm(nn.Module):
    def __init__(self, dim: int, eps: float):
        super().__init__()
        self.eps = eps if eps is not None else 1e-6
        self.weight = nn.Parameter(torch.ones(dim))

    def reset_parameters(self) -> None:
        nn.init.ones_(self.weight)

    def forward(self, x: Tensor) -> Tensor:
        return ops.rms_norm(x, self.weight, self.eps)

    def fork(self, x: Tensor) -> Tuple[Tensor, Tensor]:
        """``(norm(x), x)`` for a pre-norm residual block: pass the second value on as the residual
        so that both gradient paths meet inside the norm's backward kernel."""
        return ops.rms_norm_fork(x, self.weight, self.eps)


def ntk_scaled_base(base: float, factor: float, dim: int) -> float:
    """NTK-aware base: ``base * factor^(dim / (dim - 2))``."""
    return base * factor ** (dim / (dim - 2))


class RotaryEmbedding(nn.Module):
    """Holds the fp32 ``[max_len, dim/2, 2]`` (cos, sin) table (not saved in checkpoints).

    ``forward`` returns the handle ``(table, position_ids)`` that attention layers pass to
    ``ops.rope``; pairs are interleaved ``(x[2i], x[2i+1])`` and rotated in fp32.
    """

    def __init__(self, dim: int, max_len: int, base: float = 10000.0, rope_scaling: Optional[dict] = None):
        super().__init__()
        self.dim, self.max_len = dim, max_len
        if rope_scaling and rope_scaling.get("type") == "ntk":
            base = ntk_scaled_base(float(base), float(rope_scaling.get("factor", 1.0)), dim)
        self.base = float(base)
        self.register_buffer("cos_sin", ops.rope_table(dim, max_len, self.base), persistent=False)

    def forward(self, x: Tensor, position_ids: Optional[Tensor] = None) -> Tuple[Tensor, Optional[Tensor]]:
        if self.cos_sin.device != x.device or self.cos_sin.dtype != torch.float32:
            self.cos_sin = ops.rope_table(self.dim, self.max_len, self.base, device=x.device)
        return self.cos_sin, position_ids
