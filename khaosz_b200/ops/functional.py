"""Op layer: each function runs a hand-written sm_100a kernel for CUDA bf16 tensors and a
plain PyTorch implementation otherwise (CPU, fp32).  The PyTorch branch is the numerical
oracle the kernel tests compare against; it is never used for CUDA bf16 inputs.

Replaces the ATen/cuBLAS call sites of the reference model (``astrai/model/components/
{linear,norm,rope,mlp,attention,embedding}.py``) and its loss (``astrai/trainer/strategy.py:145-167``).
"""

from __future__ import annotations

import math
from typing import Optional, Tuple

import torch
import torch.nn.functional as F

from . import _lib
from ._lib import check, lib, ptr, stream, use_kernels

# ---------------------------------------------------------------------------------------
# GEMM
# ---------------------------------------------------------------------------------------


def _as2d(t: torch.Tensor) -> torch.Tensor:
    t2 = t.reshape(-1, t.shape[-1])
    if t2.stride(-1) != 1 or (t2.stride(0) % 8) or (t2.data_ptr() % 16):
        t2 = t2.contiguous()
    return t2


def gemm(a: torch.Tensor, b: torch.Tensor, *, a_mn: bool = False, b_mn: bool = False,
         out: Optional[torch.Tensor] = None, residual: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``C = op(A) @ op(B)^T (+ residual)`` on the tcgen05 GEMM.

    ``a_mn=False``: ``a`` is ``[M, K]``; ``a_mn=True``: ``a`` is stored ``[K, M]``.
    ``b_mn=False``: ``b`` is ``[N, K]``; ``b_mn=True``: ``b`` is stored ``[K, N]``.
    """
    M = a.shape[1] if a_mn else a.shape[0]
    K = a.shape[0] if a_mn else a.shape[1]
    N = b.shape[1] if b_mn else b.shape[0]
    Kb = b.shape[0] if b_mn else b.shape[1]
    assert K == Kb, f"inner dimensions differ: {K} vs {Kb}"
    if out is None:
        out = torch.empty((M, N), dtype=a.dtype, device=a.device)
    if not use_kernels(a):
        am = a.t() if a_mn else a
        bm = b if b_mn else b.t()
        res = am.float() @ bm.float()
        if residual is not None:
            res = res + residual.float()
        out.copy_(res.to(out.dtype))
        return out
    assert a.stride(-1) == 1 and b.stride(-1) == 1 and out.stride(-1) == 1
    epi = 0
    ldr = 0
    if residual is not None:
        assert residual.shape == out.shape and residual.stride(-1) == 1
        epi = 1
        ldr = residual.stride(0)
    # wide outputs run on CTA pairs (cta_group::2, 256x256 tiles); measured 3-5 % faster there,
    # while narrow outputs lose to the single-CTA kernel's finer wave granularity
    fn = lib().kb_gemm_bf16_pair if (N >= 4096 and M >= 512 and _lib.has("kb_gemm_bf16_pair")) else lib().kb_gemm_bf16
    check(fn(ptr(a), ptr(b), ptr(out), ptr(residual), M, N, K, a.stride(0), b.stride(0), out.stride(0), ldr,
             int(a_mn), int(b_mn), epi, stream()), "gemm_bf16")
    return out


_FP8_FORWARD = False

# A data-parallel executor that reduces gradient buckets while the backward pass is still running
# installs a callback here.  Weight gradients of the linear layers leave through the GEMM epilogue
# (``main_grad``), not through autograd's accumulation, so the layer functions themselves say when a
# weight has received its last contribution of the micro-batch: every forward use that will produce
# a weight gradient is counted, every backward use counts down.
_GRAD_READY_HOOK = None


def set_grad_ready_hook(fn) -> None:
    global _GRAD_READY_HOOK
    _GRAD_READY_HOOK = fn


def _count_use(w) -> None:
    if _GRAD_READY_HOOK is not None:
        w._kb_uses = getattr(w, "_kb_uses", 0) + 1


def _use_done(w) -> None:
    if _GRAD_READY_HOOK is not None:
        w._kb_done = getattr(w, "_kb_done", 0) + 1
        if w._kb_done >= getattr(w, "_kb_uses", 0):
            _GRAD_READY_HOOK(w)


_FP8_DGRAD = False


def set_fp8_linear(enabled: bool, dgrad: bool = False) -> None:
    """Run the forward GEMM of every bf16 linear layer in block-scaled fp8 (e4m3; 1x128
    activation scales, 128x128 weight scales, quantised on the fly from the bf16 master
    weights).  With ``dgrad`` the input-gradient GEMM runs in fp8 as well (the output gradient with
    1x128 scales along the output features, the transposed weight with 128x128 scales, cached per
    optimizer step like the forward image); weight gradients stay bf16 GEMMs into the fp32-accurate
    accumulation of the flat gradient buffer."""
    global _FP8_FORWARD, _FP8_DGRAD
    _FP8_FORWARD = bool(enabled)
    _FP8_DGRAD = bool(enabled) and bool(dgrad)


def fp8_linear_enabled() -> bool:
    return _FP8_FORWARD


# fp8 images of the bf16 master weights, valid for one weight generation: the optimizers update the
# weights in place through raw pointers (no autograd version bump), so they announce every update here
# and the 128x128-block quantisation of a weight runs once per optimizer step, not once per micro-batch.
# An entry is found by the weight's address and shape and keeps the weight alive, so that within one
# generation the address cannot be handed to another tensor; a new generation drops every entry.
_WEIGHT_GENERATION = 0
_FP8_WEIGHT_CACHE: dict = {}


def bump_weight_generation() -> None:
    global _WEIGHT_GENERATION
    _WEIGHT_GENERATION += 1
    _FP8_WEIGHT_CACHE.clear()


def _fp8_weight(w: torch.Tensor):
    from .quant import quantize_fp8_128x128

    key = (w.data_ptr(), tuple(w.shape), tuple(w.stride()))
    hit = _FP8_WEIGHT_CACHE.get(key)
    if hit is not None and hit[0] == _WEIGHT_GENERATION:
        return hit[1], hit[2]
    b8, sb = quantize_fp8_128x128(w)
    _FP8_WEIGHT_CACHE[key] = (_WEIGHT_GENERATION, b8, sb, w)
    return b8, sb


def _fp8_weight_t(w: torch.Tensor):
    """fp8 image of ``w.T`` (``[in, out]``, 128x128 scales) for the input-gradient GEMM."""
    from .quant import quantize_fp8_128x128

    key = (w.data_ptr(), tuple(w.shape), tuple(w.stride()), "t")
    hit = _FP8_WEIGHT_CACHE.get(key)
    if hit is not None and hit[0] == _WEIGHT_GENERATION:
        return hit[1], hit[2]
    b8, sb = quantize_fp8_128x128(w.t().contiguous())
    _FP8_WEIGHT_CACHE[key] = (_WEIGHT_GENERATION, b8, sb, w)
    return b8, sb


def dgrad_fp8(dy2: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """``dy2 [M, out] @ w [out, in]`` in block-scaled fp8 -> bf16 ``[M, in]``."""
    from .quant import gemm_fp8, quantize_fp8_1x128

    d8, sd = quantize_fp8_1x128(dy2)
    w8, sw = _fp8_weight_t(w)
    return gemm_fp8(d8, sd, w8, sw)


def _dgrad(dy2: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """Input gradient ``dy2 @ w`` of a linear layer with weight ``w [out, in]``."""
    if (_FP8_DGRAD and w.shape[0] % 128 == 0 and w.shape[1] % 128 == 0 and dy2.dtype == torch.bfloat16
            and _lib.has("kb_gemm_fp8")):
        return dgrad_fp8(dy2, w)
    return gemm(dy2, w, b_mn=True)


def _forward_gemm(x2: torch.Tensor, w: torch.Tensor, residual: Optional[torch.Tensor] = None) -> torch.Tensor:
    if _FP8_FORWARD and x2.shape[1] % 128 == 0 and w.shape[0] % 8 == 0 and _lib.has("kb_gemm_fp8"):
        from .quant import gemm_fp8, quantize_fp8_1x128

        a8, sa = quantize_fp8_1x128(x2)
        b8, sb = _fp8_weight(w)
        y = gemm_fp8(a8, sa, b8, sb)
        return y if residual is None else y.add_(residual)
    return gemm(x2, w, residual=residual)


class _LinearFn(torch.autograd.Function):
    """y = x W^T (+ residual); dgrad and wgrad run on the same kernel with MN-major operands."""

    @staticmethod
    def forward(ctx, x, w, residual):
        x2 = _as2d(x)
        res2 = _as2d(residual) if residual is not None else None
        y = _forward_gemm(x2, w, res2)
        ctx.save_for_backward(x2, w)
        ctx.w_ref = w
        if ctx.needs_input_grad[1]:
            _count_use(w)
        ctx.x_shape = x.shape
        ctx.has_res = residual is not None
        return y.view(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x2, w = ctx.saved_tensors
        dy2 = _as2d(dy)
        dx = dw = None
        if ctx.needs_input_grad[0]:
            dx = _dgrad(dy2, w).view(ctx.x_shape)
        if ctx.needs_input_grad[1]:
            main = getattr(ctx.w_ref, "main_grad", None)
            if main is not None:
                # accumulate straight into the flat gradient buffer (C = A^T B + C)
                gemm(dy2, x2, a_mn=True, b_mn=True, out=main, residual=main)
                ctx.w_ref.main_grad_dirty = True
                _use_done(ctx.w_ref)
            else:
                dw = gemm(dy2, x2, a_mn=True, b_mn=True)
        dres = dy if ctx.has_res else None
        return dx, dw, dres


def linear(x: torch.Tensor, w: torch.Tensor, residual: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Bias-free linear layer ``x @ w.T`` with an optional fused residual add."""
    if not use_kernels(x, w) or w.dtype != torch.bfloat16:
        y = F.linear(x, w)
        return y if residual is None else y + residual
    return _LinearFn.apply(x, w, residual)


def _adjacent(ws) -> Optional[torch.Tensor]:
    """If the weights are consecutive row blocks of one buffer return the stacked view."""
    first = ws[0]
    if not all(w.is_contiguous() and w.shape[1] == first.shape[1] and w.dtype == first.dtype for w in ws):
        return None
    expect = first.data_ptr()
    base = first.untyped_storage().data_ptr()
    for w in ws:
        # consecutive addresses inside ONE storage (separate allocations can touch by accident)
        if w.data_ptr() != expect or w.untyped_storage().data_ptr() != base:
            return None
        expect += w.numel() * w.element_size()
    rows = sum(w.shape[0] for w in ws)
    if (first.storage_offset() + rows * first.shape[1]) * first.element_size() > first.untyped_storage().nbytes():
        return None
    return first.as_strided((rows, first.shape[1]), (first.shape[1], 1), first.storage_offset())


class _MultiLinearFn(torch.autograd.Function):
    """Several bias-free linears sharing one input, computed as one GEMM over weights that
    are adjacent in memory (q/k/v and gate/up).  The weights stay separate parameters."""

    @staticmethod
    def forward(ctx, x, *ws):
        x2 = _as2d(x)
        wcat = _adjacent([w.detach() for w in ws])
        assert wcat is not None
        y = _forward_gemm(x2, wcat)
        ctx.save_for_backward(x2, wcat)
        ctx.ws = ws
        ctx.x_shape = x.shape
        for i, w in enumerate(ws):
            if ctx.needs_input_grad[i + 1]:
                _count_use(w)
        return y.view(*x.shape[:-1], wcat.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x2, wcat = ctx.saved_tensors
        dy2 = _as2d(dy)
        dx = _dgrad(dy2, wcat).view(ctx.x_shape) if ctx.needs_input_grad[0] else None
        mains = [getattr(w, "main_grad", None) for w in ctx.ws]
        need = [ctx.needs_input_grad[i + 1] for i in range(len(ctx.ws))]
        grads = [None] * len(ctx.ws)
        if any(need):
            mcat = _adjacent(mains) if all(m is not None for m in mains) and all(need) else None
            if mcat is not None:
                gemm(dy2, x2, a_mn=True, b_mn=True, out=mcat, residual=mcat)
                for w in ctx.ws:
                    w.main_grad_dirty = True
                    _use_done(w)
            else:
                dw = gemm(dy2, x2, a_mn=True, b_mn=True)
                r = 0
                for i, w in enumerate(ctx.ws):
                    if need[i]:
                        grads[i] = dw[r:r + w.shape[0]]
                    r += w.shape[0]
        return (dx, *grads)


def multi_linear(x: torch.Tensor, ws) -> torch.Tensor:
    """``cat([x @ w.T for w in ws], -1)``; one GEMM when the weights are adjacent in memory."""
    ws = list(ws)
    if use_kernels(x) and all(w.dtype == torch.bfloat16 for w in ws) and _adjacent([w.detach() for w in ws]) is not None:
        return _MultiLinearFn.apply(x, *ws)
    return torch.cat([linear(x, w) for w in ws], dim=-1)


# ---------------------------------------------------------------------------------------
# RMSNorm (+ residual)
# ---------------------------------------------------------------------------------------


class _RMSNormFn(torch.autograd.Function):
    """``fork=True`` (no ``res``) also returns ``x`` itself as a second output: the caller feeds that
    alias to the residual connection, so the gradient of the residual path arrives here and is
    added inside the backward kernel instead of by a separate accumulation pass."""

    @staticmethod
    def forward(ctx, x, res, w, eps, fork=False):
        shape = x.shape
        dim = shape[-1]
        x2 = x.reshape(-1, dim).contiguous()
        rows = x2.shape[0]
        y = torch.empty_like(x2)
        rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
        if res is not None:
            r2 = res.reshape(-1, dim).contiguous()
            s = torch.empty_like(x2)
        else:
            r2 = None
            s = None
        check(lib().kb_rmsnorm_fwd(ptr(x2), ptr(r2), ptr(w), ptr(y), ptr(s), ptr(rstd), rows, dim,
                                   float(eps), stream()), "rmsnorm_fwd")
        inp = s if s is not None else x2
        ctx.save_for_backward(inp, w, rstd)
        ctx.has_res = res is not None
        ctx.shape = shape
        if res is not None:
            return y.view(shape), s.view(shape)
        if fork:
            return y.view(shape), x.view_as(x)
        return y.view(shape), None

    @staticmethod
    def backward(ctx, dy, dsum):
        inp, w, rstd = ctx.saved_tensors
        rows, dim = inp.shape
        dy2 = dy.reshape(rows, dim).contiguous()
        ds2 = dsum.reshape(rows, dim).contiguous() if dsum is not None else None
        dx = torch.empty_like(inp)
        nparts = lib().kb_rmsnorm_bwd_partials(rows)
        partial = torch.empty((nparts, dim), dtype=torch.float32, device=inp.device)
        dw = torch.empty(dim, dtype=torch.float32, device=inp.device)
        check(lib().kb_rmsnorm_bwd(ptr(dy2), ptr(inp), ptr(w), ptr(rstd), ptr(ds2), ptr(dx), ptr(dw),
                                   ptr(partial), rows, dim, stream()), "rmsnorm_bwd")
        _lib.add_launches(1)
        dxv = dx.view(ctx.shape)
        return dxv, (dxv if ctx.has_res else None), dw.to(w.dtype), None, None


def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    if not use_kernels(x) or x.shape[-1] % 8 or x.shape[-1] > 8192:
        return F.rms_norm(x, (x.shape[-1],), w, eps)
    return _RMSNormFn.apply(x, None, w, eps)[0]


def rms_norm_fork(x: torch.Tensor, w: torch.Tensor, eps: float) -> Tuple[torch.Tensor, torch.Tensor]:
    """Returns ``(rmsnorm(x) * w, x)``; use the second value for the residual connection (see
    ``_RMSNormFn``)."""
    if not use_kernels(x) or x.shape[-1] % 8 or x.shape[-1] > 8192 or not torch.is_grad_enabled():
        return rms_norm(x, w, eps), x
    return _RMSNormFn.apply(x, None, w, eps, True)


def add_rms_norm(x: torch.Tensor, res: torch.Tensor, w: torch.Tensor, eps: float) -> Tuple[torch.Tensor, torch.Tensor]:
    """Returns ``(rmsnorm(x + res) * w, x + res)`` from one kernel."""
    if not use_kernels(x) or x.shape[-1] % 8 or x.shape[-1] > 8192:
        s = x + res
        return F.rms_norm(s, (s.shape[-1],), w, eps), s
    return _RMSNormFn.apply(x, res, w, eps)


# ---------------------------------------------------------------------------------------
# RoPE (interleaved pairs, fp32 math)
# ---------------------------------------------------------------------------------------


def rope_table(head_dim: int, max_len: int, base: float = 10000.0, device=None) -> torch.Tensor:
    """``[max_len, head_dim/2, 2]`` fp32 table of (cos, sin), computed in fp64."""
    inv = 1.0 / (base ** (torch.arange(0, head_dim, 2, dtype=torch.float64, device=device) / head_dim))
    ang = torch.outer(torch.arange(max_len, dtype=torch.float64, device=device), inv)
    return torch.stack([ang.cos(), ang.sin()], dim=-1).float().contiguous()


def _rope_torch(x: torch.Tensor, cs: torch.Tensor, pos: Optional[torch.Tensor], inverse: bool = False):
    # x: [B, S, H, D]
    B, S, H, D = x.shape
    if pos is None:
        t = cs[:S].unsqueeze(0)  # [1,S,D/2,2]
    else:
        t = cs[pos.long()]  # [B,S,D/2,2]
    cos = t[..., 0].unsqueeze(2)
    sin = t[..., 1].unsqueeze(2)
    if inverse:
        sin = -sin
    xf = x.float().reshape(B, S, H, D // 2, 2)
    a, b = xf[..., 0], xf[..., 1]
    out = torch.stack([a * cos - b * sin, a * sin + b * cos], dim=-1)
    return out.reshape(B, S, H, D).to(x.dtype)


def _rope_kernel(x, cs, pos, n_heads, inverse):
    # x: [B, S, Hx, D] possibly a view into a packed projection buffer; rotates the first n_heads
    B, S, Hx, D = x.shape
    assert x.stride(3) == 1 and x.stride(2) == D and x.stride(0) == S * x.stride(1)
    pos32 = None
    if pos is not None:
        pos32 = pos.to(torch.int32).expand(B, S).contiguous()
    check(lib().kb_rope(ptr(x), ptr(x), ptr(cs), ptr(pos32), B * S, S, n_heads, D, x.stride(1),
                        int(inverse), stream()), "rope")


class _RopeFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, cs, pos, n_heads):
        y = x.clone(memory_format=torch.contiguous_format)
        _rope_kernel(y, cs, pos, n_heads, False)
        ctx.cs, ctx.pos, ctx.n_heads = cs, pos, n_heads
        return y

    @staticmethod
    def backward(ctx, dy):
        dx = dy.clone(memory_format=torch.contiguous_format)
        _rope_kernel(dx, ctx.cs, ctx.pos, ctx.n_heads, True)
        return dx, None, None, None


def rope(x: torch.Tensor, cs: torch.Tensor, pos: Optional[torch.Tensor] = None,
         n_heads: Optional[int] = None) -> torch.Tensor:
    """Rotate the first ``n_heads`` heads of ``x [B,S,H,D]`` (all heads by default)."""
    H = x.shape[2]
    n_heads = H if n_heads is None else n_heads
    if not use_kernels(x) or x.shape[-1] % 8:
        if n_heads == H:
            return _rope_torch(x, cs, pos)
        return torch.cat([_rope_torch(x[:, :, :n_heads], cs, pos), x[:, :, n_heads:]], dim=2)
    return _RopeFn.apply(x, cs, pos, n_heads)


# ---------------------------------------------------------------------------------------
# SwiGLU
# ---------------------------------------------------------------------------------------


class _SwiGLUFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gu):
        F2 = gu.shape[-1]
        gu2 = gu.reshape(-1, F2).contiguous()
        h = torch.empty((gu2.shape[0], F2 // 2), dtype=gu.dtype, device=gu.device)
        check(lib().kb_swiglu_fwd(ptr(gu2), ptr(h), gu2.shape[0], F2 // 2, stream()), "swiglu_fwd")
        ctx.save_for_backward(gu2)
        ctx.shape = gu.shape
        return h.view(*gu.shape[:-1], F2 // 2)

    @staticmethod
    def backward(ctx, dh):
        (gu2,) = ctx.saved_tensors
        dh2 = dh.reshape(gu2.shape[0], -1).contiguous()
        dgu = torch.empty_like(gu2)
        check(lib().kb_swiglu_bwd(ptr(gu2), ptr(dh2), ptr(dgu), gu2.shape[0], gu2.shape[1] // 2, stream()),
              "swiglu_bwd")
        return dgu.view(ctx.shape)


class _LinearSwiGLUFn(torch.autograd.Function):
    """``h = up(x) * silu(gate(x))`` from ONE kernel: the gate|up GEMM over the adjacent weights with
    the SwiGLU in its epilogue (``kb_gemm_swiglu_bf16``).  The epilogue also writes ``[gate | up]``,
    which the backward pass needs; what disappears is the separate SwiGLU launch and its re-read of
    the ``[tokens, 2F]`` projection."""

    @staticmethod
    def forward(ctx, x, w_gate, w_up):
        x2 = _as2d(x)
        wcat = _adjacent([w_gate.detach(), w_up.detach()])
        assert wcat is not None
        M, K = x2.shape
        Fh = w_gate.shape[0]
        gu = torch.empty((M, 2 * Fh), dtype=x2.dtype, device=x2.device)
        h = torch.empty((M, Fh), dtype=x2.dtype, device=x2.device)
        check(lib().kb_gemm_swiglu_bf16(ptr(x2), ptr(wcat), ptr(gu), ptr(h), M, Fh, K, x2.stride(0), wcat.stride(0),
                                        gu.stride(0), h.stride(0), 0, stream()), "gemm_swiglu")
        ctx.save_for_backward(x2, wcat, gu)
        ctx.ws = (w_gate, w_up)
        ctx.x_shape = x.shape
        for i, w in enumerate(ctx.ws):
            if ctx.needs_input_grad[i + 1]:
                _count_use(w)
        return h.view(*x.shape[:-1], Fh)

    @staticmethod
    def backward(ctx, dh):
        x2, wcat, gu = ctx.saved_tensors
        dh2 = dh.reshape(gu.shape[0], -1).contiguous()
        dgu = torch.empty_like(gu)
        check(lib().kb_swiglu_bwd(ptr(gu), ptr(dh2), ptr(dgu), gu.shape[0], gu.shape[1] // 2, stream()), "swiglu_bwd")
        dx = gemm(dgu, wcat, b_mn=True).view(ctx.x_shape) if ctx.needs_input_grad[0] else None
        grads = [None, None]
        need = [ctx.needs_input_grad[1], ctx.needs_input_grad[2]]
        if any(need):
            mains = [getattr(w, "main_grad", None) for w in ctx.ws]
            mcat = _adjacent(mains) if all(m is not None for m in mains) and all(need) else None
            if mcat is not None:
                gemm(dgu, x2, a_mn=True, b_mn=True, out=mcat, residual=mcat)
                for w in ctx.ws:
                    w.main_grad_dirty = True
                    _use_done(w)
            else:
                dw = gemm(dgu, x2, a_mn=True, b_mn=True)
                Fh = ctx.ws[0].shape[0]
                grads = [dw[:Fh] if need[0] else None, dw[Fh:] if need[1] else None]
        return (dx, *grads)


def linear_swiglu(x: torch.Tensor, w_gate: torch.Tensor, w_up: torch.Tensor) -> torch.Tensor:
    """``(x @ w_up.T) * silu(x @ w_gate.T)``; one fused kernel when the two weights are adjacent in
    memory (gate first), bf16, on CUDA (reference: ``astrai/model/components/mlp.py:25-26``)."""
    Fh = w_gate.shape[0]
    if (use_kernels(x) and w_gate.dtype == torch.bfloat16 and w_up.dtype == torch.bfloat16 and Fh % 8 == 0
            and w_up.shape == w_gate.shape and not _FP8_FORWARD and _lib.has("kb_gemm_swiglu_bf16")
            and _adjacent([w_gate.detach(), w_up.detach()]) is not None):
        return _LinearSwiGLUFn.apply(x, w_gate, w_up)
    return swiglu(multi_linear(x, (w_gate, w_up)))


def swiglu(gu: torch.Tensor) -> torch.Tensor:
    """``up * silu(gate)`` for ``gu = [gate | up]`` concatenated on the last dimension."""
    Fh = gu.shape[-1] // 2
    if not use_kernels(gu) or Fh % 8:
        g, u = gu[..., :Fh], gu[..., Fh:]
        return u * F.silu(g)
    return _SwiGLUFn.apply(gu)


# ---------------------------------------------------------------------------------------
# Cross entropy / token log-probs
# ---------------------------------------------------------------------------------------


class _CEFn(torch.autograd.Function):
    """Per-row loss (mode 0) or target log-prob (mode 1); the backward overwrites the logits
    buffer with the gradient (the logits are dead after the loss)."""

    @staticmethod
    def forward(ctx, logits, targets, smoothing, ignore_index, mode):
        V = logits.shape[-1]
        z = logits.reshape(-1, V)
        if z.stride(-1) != 1 or z.stride(0) % 8:
            z = z.contiguous()
        t = targets.reshape(-1).to(torch.int64).contiguous()
        rows = z.shape[0]
        out = torch.empty(rows, dtype=torch.float32, device=z.device)
        lse = torch.empty(rows, dtype=torch.float32, device=z.device)
        loss_p = ptr(out) if mode == 0 else None
        logp_p = ptr(out) if mode == 1 else None
        check(lib().kb_ce_fwd(ptr(z), ptr(t), loss_p, ptr(lse), logp_p, rows, V, z.stride(0),
                              float(smoothing), int(ignore_index), stream()), "ce_fwd")
        ctx.save_for_backward(z, t, lse)
        ctx.args = (float(smoothing), int(ignore_index), int(mode), logits.shape)
        return out

    @staticmethod
    def backward(ctx, g):
        z, t, lse = ctx.saved_tensors
        smoothing, ignore_index, mode, shape = ctx.args
        g = g.to(torch.float32).contiguous()
        rows, V = z.shape
        dz = z  # in place: the forward activations are not needed again
        check(lib().kb_ce_bwd(ptr(z), ptr(t), ptr(lse), ptr(g), ptr(dz), rows, V, z.stride(0), smoothing,
                              ignore_index, mode, stream()), "ce_bwd")
        return dz.view(shape), None, None, None, None


def cross_entropy_rows(logits: torch.Tensor, targets: torch.Tensor, label_smoothing: float = 0.0,
                       ignore_index: int = -100) -> torch.Tensor:
    """Per-row label-smoothed NLL (fp32), zero where ``targets == ignore_index``."""
    if not use_kernels(logits):
        return F.cross_entropy(logits.reshape(-1, logits.shape[-1]).float(), targets.reshape(-1),
                               reduction="none", label_smoothing=label_smoothing, ignore_index=ignore_index)
    return _CEFn.apply(logits, targets, label_smoothing, ignore_index, 0)


def cross_entropy(logits: torch.Tensor, targets: torch.Tensor, label_smoothing: float = 0.0,
                  ignore_index: int = -100) -> torch.Tensor:
    """Mean label-smoothed cross entropy over the non-ignored targets (``F.cross_entropy``
    semantics, fp32 math, no fp32 copy of the logits).  A batch whose targets are all ignored gives
    0 (``F.cross_entropy`` gives NaN there), so a fully masked micro-batch cannot poison a run."""
    rows = cross_entropy_rows(logits, targets, label_smoothing, ignore_index)
    count = (targets.reshape(-1) != ignore_index).sum().clamp_min(1)
    return rows.sum() / count


def token_logprobs(logits: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
    """``log_softmax(logits)[..., targets]`` with the shape of ``targets`` (fp32)."""
    if not use_kernels(logits):
        lp = torch.log_softmax(logits.float(), dim=-1)
        return lp.gather(-1, targets.unsqueeze(-1)).squeeze(-1)
    return _CEFn.apply(logits, targets, 0.0, -100, 1).view(targets.shape)


# ---------------------------------------------------------------------------------------
# Embedding
# ---------------------------------------------------------------------------------------


class _EmbeddingFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, ids, table):
        flat = ids.reshape(-1).to(torch.int64).contiguous()
        out = torch.empty((flat.numel(), table.shape[1]), dtype=table.dtype, device=table.device)
        check(lib().kb_embedding_fwd(ptr(table), ptr(flat), ptr(out), flat.numel(), table.shape[1],
                                     table.shape[0], stream()), "embedding_fwd")
        ctx.save_for_backward(flat)
        ctx.table_shape = table.shape
        ctx.w_ref = table
        return out.view(*ids.shape, table.shape[1])

    @staticmethod
    def backward(ctx, dy):
        (flat,) = ctx.saved_tensors
        V, D = ctx.table_shape
        dy2 = dy.reshape(-1, D).contiguous()
        dt = torch.zeros((V, D), dtype=torch.float32, device=dy.device)
        check(lib().kb_embedding_bwd(ptr(dy2), ptr(flat), ptr(dt), flat.numel(), D, V, stream()),
              "embedding_bwd")
        main = getattr(ctx.w_ref, "main_grad", None)
        if main is not None:
            main.add_(dt)
            ctx.w_ref.main_grad_dirty = True
            return None, None
        return None, dt.to(dy.dtype)


def embedding(ids: torch.Tensor, table: torch.Tensor) -> torch.Tensor:
    if not use_kernels(table) or table.shape[1] % 8:
        return F.embedding(ids, table)
    return _EmbeddingFn.apply(ids, table)


# ---------------------------------------------------------------------------------------
# Attention (see attention.py for the kernels' wrappers)
# ---------------------------------------------------------------------------------------


def sdpa_reference(q, k, v, causal: bool, scale: Optional[float] = None, mask=None):
    """fp32 softmax attention on ``[B,S,H,D]`` tensors with GQA broadcast; the oracle."""
    B, S, H, D = q.shape
    Hkv = k.shape[2]
    T = k.shape[1]
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    qf = q.float().permute(0, 2, 1, 3)
    kf = k.float().permute(0, 2, 1, 3).repeat_interleave(H // Hkv, dim=1)
    vf = v.float().permute(0, 2, 1, 3).repeat_interleave(H // Hkv, dim=1)
    s = qf @ kf.transpose(-1, -2) * scale
    if causal:
        cm = torch.ones(S, T, dtype=torch.bool, device=q.device).tril(T - S)
        s = s.masked_fill(~cm, float("-inf"))
    if mask is not None:
        s = s + mask.float()
    p = torch.softmax(s, dim=-1)
    return (p @ vf).permute(0, 2, 1, 3).to(q.dtype)
