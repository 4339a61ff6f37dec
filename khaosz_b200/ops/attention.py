"""Attention ops.

* :func:`rope_attention_packed` — training / prefill path: RoPE applied in place on the packed
  ``[B,S,H+2Hkv,D]`` projection buffer, then causal flash attention (tcgen05 kernels for
  ``D == 128``) reading q/k/v straight out of that buffer; the backward writes one packed
  gradient buffer and un-rotates it in place.
* :func:`attention` — same kernels for unpacked ``[B,S,H,D]`` tensors (heads narrower than 128 run
  zero-padded); every other configuration (fp32, CPU, explicit masks, cross lengths) takes the
  plain softmax attention with GQA broadcast, which is also the oracle of the tests.

Replaces ``repeat_kv`` + permutes + ``F.scaled_dot_product_attention`` of the reference
(``astrai/model/components/attention.py:95-103``).
"""

from __future__ import annotations

import math
from typing import Optional

import torch
import torch.nn.functional as F

from . import _lib
from ._lib import check, lib, ptr, stream
from .functional import _rope_kernel, _rope_torch, sdpa_reference

FLASH_HEAD_DIM = 128


def flash_available() -> bool:
    return _lib.available() and _lib.has("kb_flash_fwd")


def fused_ok(qkv: torch.Tensor, head_dim: int) -> bool:
    return qkv.is_cuda and qkv.dtype == torch.bfloat16 and head_dim == FLASH_HEAD_DIM and qkv.is_contiguous()


def _flash_fwd(q, k, v, causal, scale):
    """q [B,S,H,D], k/v [B,S,Hkv,D] views with unit inner stride and a common row pitch."""
    B, S, H, D = q.shape
    T, Hkv = k.shape[1], k.shape[2]
    o = torch.empty((B, S, H, D), dtype=q.dtype, device=q.device)
    lse = torch.empty((B, H, S), dtype=torch.float32, device=q.device)
    if T == S:
        check(lib().kb_flash_fwd(ptr(q), ptr(k), ptr(v), ptr(o), ptr(lse), B, S, H, Hkv, D, q.stride(1), k.stride(1),
                                 v.stride(1), o.stride(1), float(scale), int(causal), stream()), "flash_fwd")
    else:   # the queries are the last S of T positions (prefill behind a cached prefix)
        assert k.stride(0) == T * k.stride(1) and v.stride(0) == T * v.stride(1)
        check(lib().kb_flash_fwd_rect(ptr(q), ptr(k), ptr(v), ptr(o), ptr(lse), B, S, T, H, Hkv, D, q.stride(1),
                                      k.stride(1), v.stride(1), o.stride(1), float(scale), int(causal), stream()),
              "flash_fwd_rect")
    return o, lse


def _flash_bwd(q, k, v, o, do, lse, dq, dk, dv, causal, scale):
    B, S, H, D = q.shape
    Hkv = k.shape[2]
    delta = torch.empty((B, H, S), dtype=torch.float32, device=q.device)
    check(lib().kb_flash_bwd(ptr(q), ptr(k), ptr(v), ptr(o), ptr(do), ptr(lse), ptr(delta), ptr(dq), ptr(dk), ptr(dv),
                             B, S, H, Hkv, D, q.stride(1), k.stride(1), v.stride(1), o.stride(1), do.stride(1),
                             dq.stride(1), dk.stride(1), dv.stride(1), float(scale), int(causal), stream()),
          "flash_bwd")
    _lib.add_launches(2)


class _RopeAttnPackedFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, qkv, cs, pos, H, Hkv, causal):
        B, S, _, D = qkv.shape
        scale = 1.0 / math.sqrt(D)
        # in place through the raw pointer: qkv is a fresh GEMM output that nothing else reads,
        # and the projection's backward does not need its own output
        _rope_kernel(qkv, cs, pos, H + Hkv, False)
        q, k, v = qkv[:, :, :H], qkv[:, :, H:H + Hkv], qkv[:, :, H + Hkv:]
        o, lse = _flash_fwd(q, k, v, causal, scale)
        ctx.save_for_backward(qkv, o, lse)
        ctx.meta = (cs, pos, H, Hkv, causal, scale)
        return o

    @staticmethod
    def backward(ctx, do):
        qkv, o, lse = ctx.saved_tensors
        cs, pos, H, Hkv, causal, scale = ctx.meta
        do = do.contiguous()
        dqkv = torch.empty_like(qkv)
        q, k, v = qkv[:, :, :H], qkv[:, :, H:H + Hkv], qkv[:, :, H + Hkv:]
        dq, dk, dv = dqkv[:, :, :H], dqkv[:, :, H:H + Hkv], dqkv[:, :, H + Hkv:]
        _flash_bwd(q, k, v, o, do, lse, dq, dk, dv, causal, scale)
        _rope_kernel(dqkv, cs, pos, H + Hkv, True)
        return dqkv, None, None, None, None, None


def rope_attention_packed(qkv: torch.Tensor, cs: torch.Tensor, pos: Optional[torch.Tensor], H: int, Hkv: int,
                          causal: bool = True) -> torch.Tensor:
    """RoPE + attention on a packed projection buffer ``[B,S,H+2Hkv,D]`` -> ``[B,S,H,D]``."""
    if flash_available():
        return _RopeAttnPackedFn.apply(qkv, cs, pos, H, Hkv, causal)
    from .functional import rope

    qk = rope(qkv[:, :, :H + Hkv], cs, pos)
    return attention(qk[:, :, :H], qk[:, :, H:], qkv[:, :, H + Hkv:], causal=causal)


class _FlashFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, causal, scale):
        q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
        o, lse = _flash_fwd(q, k, v, causal, scale)
        ctx.save_for_backward(q, k, v, o, lse)
        ctx.meta = (causal, scale)
        return o

    @staticmethod
    def backward(ctx, do):
        q, k, v, o, lse = ctx.saved_tensors
        causal, scale = ctx.meta
        dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
        _flash_bwd(q, k, v, o, do.contiguous(), lse, dq, dk, dv, causal, scale)
        return dq, dk, dv, None, None


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, causal: bool = True,
              mask: Optional[torch.Tensor] = None, scale: Optional[float] = None) -> torch.Tensor:
    """Softmax attention on ``[B,S,H,D]`` / ``[B,T,Hkv,D]`` tensors.

    ``mask`` is an additive ``[B,1,S,T]`` (or broadcastable) tensor; with a mask ``causal`` is
    ignored exactly like the reference does.
    """
    B, S, H, D = q.shape
    T, Hkv = k.shape[1], k.shape[2]
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    # S < T (queries behind a cached prefix) runs the forward kernel only: serving needs no gradient
    lengths_ok = S == T or (S < T and not (torch.is_grad_enabled() and (q.requires_grad or k.requires_grad or v.requires_grad))
                            and _lib.has("kb_flash_fwd_rect"))
    if (mask is None and lengths_ok and q.is_cuda and q.dtype == torch.bfloat16 and D == FLASH_HEAD_DIM
            and v.shape[-1] == D and H % Hkv == 0 and flash_available()):
        if S != T:
            return _flash_fwd(q.contiguous(), k.contiguous(), v.contiguous(), bool(causal), scale)[0]
        return _FlashFn.apply(q, k, v, bool(causal), scale)
    if (mask is None and lengths_ok and q.is_cuda and q.dtype == torch.bfloat16 and D < FLASH_HEAD_DIM and D % 8 == 0
            and v.shape[-1] == D and H % Hkv == 0 and flash_available()):
        # smaller heads (e.g. 64, the reference's benchmark model) ride the same kernels zero-padded to
        # 128: the extra columns add nothing to q.k and produce zero output columns, the softmax scale
        # stays that of the real width; twice the tensor work of a native kernel, but no materialised
        # K/V repeat and no score matrix
        pad = FLASH_HEAD_DIM - D
        if S != T:
            return _flash_fwd(F.pad(q, (0, pad)), F.pad(k, (0, pad)), F.pad(v, (0, pad)), bool(causal), scale)[0][..., :D]
        out = _FlashFn.apply(F.pad(q, (0, pad)), F.pad(k, (0, pad)), F.pad(v, (0, pad)), bool(causal), scale)
        return out[..., :D]
    qh, kh, vh = q.permute(0, 2, 1, 3), k.permute(0, 2, 1, 3), v.permute(0, 2, 1, 3)
    if Hkv != H and kh.shape[1] != 1:
        rep = H // Hkv
        kh, vh = kh.repeat_interleave(rep, dim=1), vh.repeat_interleave(rep, dim=1)
    if mask is not None:
        out = F.scaled_dot_product_attention(qh, kh, vh, attn_mask=mask.to(qh.dtype), scale=scale)
    elif causal and S != T:
        cm = torch.ones(S, T, dtype=torch.bool, device=q.device).tril(T - S)
        out = F.scaled_dot_product_attention(qh, kh, vh, attn_mask=cm, scale=scale)
    else:
        out = F.scaled_dot_product_attention(qh, kh, vh, is_causal=bool(causal), scale=scale)
    return out.permute(0, 2, 1, 3)


__all__ = ["attention", "rope_attention_packed", "fused_ok", "flash_available", "sdpa_reference", "_rope_torch"]
