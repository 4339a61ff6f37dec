"""Weight-only int8 inference: per-output-channel symmetric quantisation and the linear layer
that runs on the int8-weight tcgen05 GEMM (weights stay int8 in HBM, are widened to bf16 inside
the SM, the channel scale is applied to the fp32 accumulator).  Not present in the reference;
used by the int8 serving configuration."""

from __future__ import annotations

from typing import Optional, Tuple

import torch
import torch.nn as nn

from . import _lib
from ._lib import check, lib, ptr, stream


def quantize_w8(weight: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """``weight [N, K]`` -> ``(int8 [N, K], fp32 scale [N])`` with ``w ~= q * scale[:, None]``."""
    N, K = weight.shape
    if weight.is_cuda and weight.dtype == torch.bfloat16 and _lib.has("kb_quant_w8"):
        w = weight.contiguous()
        q = torch.empty((N, K), dtype=torch.int8, device=w.device)
        scale = torch.empty(N, dtype=torch.float32, device=w.device)
        check(lib().kb_quant_w8(ptr(w), ptr(q), ptr(scale), N, K, stream()), "quant_w8")
        return q, scale
    wf = weight.float()
    amax = wf.abs().amax(dim=1)
    scale = torch.where(amax > 0, amax / 127.0, torch.ones_like(amax))
    q = torch.clamp(torch.round(wf / scale[:, None]), -127, 127).to(torch.int8)
    return q, scale


def linear_w8(x: torch.Tensor, q: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    """``x @ (q * scale[:, None]).T``."""
    N, K = q.shape
    if (x.is_cuda and x.dtype == torch.bfloat16 and K % 16 == 0 and N % 8 == 0 and _lib.has("kb_gemm_w8")):
        x2 = x.reshape(-1, K)
        if x2.stride(-1) != 1 or x2.stride(0) % 8 or x2.data_ptr() % 16:
            x2 = x2.contiguous()
        out = torch.empty((x2.shape[0], N), dtype=x.dtype, device=x.device)
        check(lib().kb_gemm_w8(ptr(x2), ptr(q), ptr(scale), ptr(out), x2.shape[0], N, K, x2.stride(0), q.stride(0),
                               out.stride(0), stream()), "gemm_w8")
        return out.view(*x.shape[:-1], N)
    w = q.to(x.dtype) * scale.to(x.dtype)[:, None]
    return x @ w.t()


class Int8Linear(nn.Module):
    """Drop-in for the bias-free ``Linear`` at inference time."""

    def __init__(self, weight: torch.Tensor):
        super().__init__()
        q, scale = quantize_w8(weight.detach())
        self.register_buffer("qweight", q)
        self.register_buffer("scale", scale)
        self.in_dim, self.out_dim = weight.shape[1], weight.shape[0]

    def forward(self, x: torch.Tensor, residual: Optional[torch.Tensor] = None) -> torch.Tensor:
        y = linear_w8(x, self.qweight, self.scale)
        return y if residual is None else y + residual


def quantize_model_int8(model: nn.Module, skip=("lm_head",)) -> int:
    """Replace every bias-free ``Linear`` (except ``skip``) by :class:`Int8Linear`; returns the
    number of layers converted."""
    from ..models.components.layers import Linear

    count = 0
    for name, module in list(model.named_modules()):
        for child_name, child in list(module.named_children()):
            if type(child) is Linear and child.bias is None and child_name not in skip:
                setattr(module, child_name, Int8Linear(child.weight))
                count += 1
    return count
