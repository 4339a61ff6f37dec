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


def int8_multi_linear(x: torch.Tensor, mods) -> Optional[torch.Tensor]:
    """``cat([m(x) for m in mods], -1)`` as ONE int8 GEMM when every module is an ``Int8Linear`` of the
    same input width (q/k/v, gate/up): the quantised rows and scales are stacked once and cached on
    the first module.  Returns ``None`` when the modules do not qualify."""
    mods = list(mods)
    if not all(type(m) is Int8Linear for m in mods) or len({m.in_dim for m in mods}) != 1:
        return None
    first = mods[0]
    packed = getattr(first, "_packed", None)
    if packed is None or packed[2] != tuple(id(m) for m in mods):
        q = torch.cat([m.qweight for m in mods], dim=0).contiguous()
        sc = torch.cat([m.scale for m in mods], dim=0).contiguous()
        packed = first._packed = (q, sc, tuple(id(m) for m in mods))
    return linear_w8(x, packed[0], packed[1])


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


# ---------------------------------------------------------------------------------------
# Block-scaled fp8 (e4m3): 1x128 activation scales, 128x128 weight scales
# ---------------------------------------------------------------------------------------
FP8_MAX = 448.0


def _fp8_kernels(t: torch.Tensor) -> bool:
    return t.is_cuda and t.dtype == torch.bfloat16 and _lib.has("kb_gemm_fp8")


def quantize_fp8_1x128(x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """``x [M, K]`` -> ``(e4m3 bytes [M, K] as uint8, fp32 scale [M, K/128])``; ``K % 128 == 0``."""
    M, K = x.shape
    assert K % 128 == 0
    if _fp8_kernels(x):
        x = x if x.stride(-1) == 1 else x.contiguous()
        q = torch.empty((M, K), dtype=torch.uint8, device=x.device)
        s = torch.empty((M, K // 128), dtype=torch.float32, device=x.device)
        check(lib().kb_quant_fp8_1x128(ptr(x), ptr(q), ptr(s), M, K, x.stride(0), stream()), "quant_fp8_1x128")
        return q, s
    blocks = x.float().reshape(M, K // 128, 128)
    amax = blocks.abs().amax(dim=-1)
    s = torch.where(amax > 0, amax / FP8_MAX, torch.ones_like(amax))
    q = (blocks / s[..., None]).reshape(M, K).to(torch.float8_e4m3fn).view(torch.uint8)
    return q, s


def quantize_fp8_128x128(w: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """``w [N, K]`` -> ``(e4m3 bytes [N, K], fp32 scale [ceil(N/128), K/128])``."""
    N, K = w.shape
    assert K % 128 == 0
    nb = (N + 127) // 128
    if _fp8_kernels(w):
        w = w if w.stride(-1) == 1 else w.contiguous()
        q = torch.empty((N, K), dtype=torch.uint8, device=w.device)
        s = torch.empty((nb, K // 128), dtype=torch.float32, device=w.device)
        check(lib().kb_quant_fp8_128x128(ptr(w), ptr(q), ptr(s), N, K, w.stride(0), stream()), "quant_fp8_128x128")
        return q, s
    wf = torch.zeros((nb * 128, K), dtype=torch.float32, device=w.device)
    wf[:N] = w.float()
    blocks = wf.reshape(nb, 128, K // 128, 128)
    amax = blocks.abs().amax(dim=(1, 3))
    s = torch.where(amax > 0, amax / FP8_MAX, torch.ones_like(amax))
    q = (blocks / s[:, None, :, None]).reshape(nb * 128, K)[:N].to(torch.float8_e4m3fn).view(torch.uint8)
    return q, s


def dequantize_fp8(q: torch.Tensor, scale: torch.Tensor, weight: bool) -> torch.Tensor:
    """fp32 reconstruction (the oracle of the GEMM test)."""
    v = q.view(torch.float8_e4m3fn).float()
    R, K = v.shape
    if weight:
        s = scale.repeat_interleave(128, dim=0)[:R].repeat_interleave(128, dim=1)
    else:
        s = scale.repeat_interleave(128, dim=1)
    return v * s


def gemm_fp8(a8: torch.Tensor, sa: torch.Tensor, b8: torch.Tensor, sb: torch.Tensor) -> torch.Tensor:
    """``dequant(a8, sa) @ dequant(b8, sb).T`` -> bf16 ``[M, N]``."""
    M, K = a8.shape
    N = b8.shape[0]
    if a8.is_cuda and _lib.has("kb_gemm_fp8") and N % 8 == 0:
        out = torch.empty((M, N), dtype=torch.bfloat16, device=a8.device)
        check(lib().kb_gemm_fp8(ptr(a8), ptr(b8), ptr(sa), ptr(sb), ptr(out), M, N, K, a8.stride(0), b8.stride(0),
                                out.stride(0), stream()), "gemm_fp8")
        return out
    return (dequantize_fp8(a8, sa, False) @ dequantize_fp8(b8, sb, True).t()).to(torch.bfloat16)


class _Fp8LinearFn(torch.autograd.Function):
    """Forward in block-scaled fp8 from bf16 master weights; backward in bf16."""

    @staticmethod
    def forward(ctx, x, w):
        x2 = x.reshape(-1, x.shape[-1])
        a8, sa = quantize_fp8_1x128(x2)
        b8, sb = quantize_fp8_128x128(w)
        ctx.save_for_backward(x2, w)
        ctx.shape = x.shape
        return gemm_fp8(a8, sa, b8, sb).view(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, dy):
        from .functional import gemm

        x2, w = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1]).contiguous()
        dx = gemm(dy2, w, b_mn=True).view(ctx.shape)
        dw = gemm(dy2, x2.contiguous(), a_mn=True, b_mn=True)
        return dx, dw


def linear_fp8(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """``x @ w.T`` with e4m3 operands (1x128 / 128x128 scales) and bf16 master weights."""
    if x.shape[-1] % 128:
        return torch.nn.functional.linear(x, w)
    return _Fp8LinearFn.apply(x, w)
