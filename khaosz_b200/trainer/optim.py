"""Optimizers.

``FusedAdamW``: AdamW over the executors' flat buffers.  On CUDA bf16 the whole model (or this
rank's shard of it) is updated by one kernel launch that also applies the gradient scale and
the global-norm clip factor read from device memory (no host synchronisation); elsewhere the
same arithmetic runs as plain PyTorch and matches ``torch.optim.AdamW``.  Moments are fp32.
Replaces ``torch.optim.AdamW(fused=True)`` + ``clip_grad_norm_`` of the reference training
script (``scripts/tools/train.py:197-198``, ``astrai/trainer/train_callback.py:79-89``).

``Muon``: momentum + Newton-Schulz orthogonalised updates for matrices, AdamW for vectors
(reference: ``astrai/trainer/optim.py:5-143``).
"""

from __future__ import annotations

import math
from typing import Any, Dict, Optional, Tuple

import torch
import torch.distributed as dist
from torch.optim import Optimizer

from ..ops import _lib
from ..ops._lib import check, lib, ptr, stream


class FusedAdamW(Optimizer):
    def __init__(self, params, lr: float = 1e-3, betas: Tuple[float, float] = (0.9, 0.999), eps: float = 1e-8,
                 weight_decay: float = 1e-2):
        super().__init__(params, dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay))
        self._flat = None
        self._shard: Optional[Tuple[int, int]] = None
        self._reducer = None
        self._clip: Optional[float] = None
        self._step_count = 0
        self._m: Optional[torch.Tensor] = None
        self._v: Optional[torch.Tensor] = None
        self._lr_step_dev: Optional[torch.Tensor] = None
        self._gnorm_sq: Optional[torch.Tensor] = None
        self.last_grad_norm: Optional[torch.Tensor] = None
        self._norm_fn = None
        self._layout = None

    def set_layout(self, owned_ranges) -> None:
        """``owned_ranges(rank) -> [(dense offset, local offset, n)]``: which pieces of the dense flat
        vector the local vectors of ``rank`` hold (executors that shard block by block)."""
        self._layout = owned_ranges

    def set_norm_fn(self, fn) -> None:
        """``fn() -> device scalar`` with the global squared gradient norm; executors whose
        parameters are partly sharded and partly replicated (tensor parallel) install it."""
        self._norm_fn = fn

    # -- wiring done by the executors -------------------------------------------------------
    def attach_flat(self, flat, shard: Optional[Tuple[int, int]] = None, allocate: bool = True) -> None:
        """Operate on ``flat.data`` / ``flat.grad`` (optionally only ``[offset, offset+n)``)."""
        mine = {id(p) for g in self.param_groups for p in g["params"]}
        trainable = {id(p) for p in flat.params if p.requires_grad}
        if len(self.param_groups) != 1 or mine != trainable or len(trainable) != len(flat.params):
            return  # partial coverage (e.g. LoRA) keeps the per-parameter path
        self._flat, self._shard = flat, shard
        off, n = shard if shard is not None else (0, flat.numel)
        dev = flat.data.device
        if allocate:
            self._m = torch.zeros(n, dtype=torch.float32, device=dev)
            self._v = torch.zeros(n, dtype=torch.float32, device=dev)
        self._gnorm_sq = torch.zeros(1, dtype=torch.float32, device=dev)
        if dev.type == "cuda":
            self._lr_step_dev = torch.zeros(2, dtype=torch.float32, device=dev)

    def attach_reducer(self, reducer) -> None:
        """A gradient reducer that fuses the AdamW update into its collective kernel; the
        moments live with the reducer and cover this rank's slice only."""
        self._reducer = reducer
        if self._flat is not None:
            self._m, self._v, self._shard = reducer.moments()

    def fused_clip(self, max_norm: Optional[float]) -> None:
        """Clip to ``max_norm`` (global L2 norm over all ranks' shards) inside the next step."""
        self._clip = max_norm

    # -- step ---------------------------------------------------------------------------------
    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        if self._flat is not None:
            self._step_flat()
        else:
            self._step_per_param()
        self._clip = None
        from ..ops.functional import bump_weight_generation

        bump_weight_generation()    # cached fp8 images of the weights are stale now
        return loss

    def _global_norm_sq(self, g: torch.Tensor) -> torch.Tensor:
        sq = self._gnorm_sq
        sq.zero_()
        if g.is_cuda and g.dtype == torch.bfloat16:
            check(lib().kb_sumsq_bf16(ptr(g), g.numel(), ptr(sq), stream()), "sumsq")
        else:
            sq += g.float().pow(2).sum()
        if self._shard is not None and dist.is_initialized():
            dist.all_reduce(sq)
        return sq

    def _step_flat(self) -> None:
        group = self.param_groups[0]
        flat = self._flat
        off, n = self._shard if self._shard is not None else (0, flat.numel)
        p, g = flat.data[off:off + n], flat.grad[off:off + n]
        self._step_count += 1
        beta1, beta2 = group["betas"]
        lr, eps, wd = group["lr"], group["eps"], group["weight_decay"]
        clip = self._clip if self._clip and self._clip > 0 else None
        if self._reducer is not None and self._reducer.fuses_optimizer:
            self._reducer.fused_step(self, lr, beta1, beta2, eps, wd, clip, self._step_count)
            return
        gn = None
        if clip is not None:
            gn = self._norm_fn().reshape(1).float() if self._norm_fn is not None else self._global_norm_sq(g)
        if gn is not None:
            self.last_grad_norm = gn.sqrt()
        if p.is_cuda and p.dtype == torch.bfloat16:
            _lib.set_device_floats(self._lr_step_dev, lr, self._step_count)
            check(lib().kb_adamw_bf16(ptr(p), ptr(g), ptr(self._m), ptr(self._v), n, ptr(self._lr_step_dev),
                                      beta1, beta2, eps, wd, 1.0, ptr(gn) if gn is not None else None,
                                      float(clip or 0.0), stream()), "adamw")
            return
        gf = g.float()
        if gn is not None:
            gf = gf * torch.clamp(clip / (gn.sqrt() + 1e-6), max=1.0)
        self._adamw_math(p, gf, self._m, self._v, lr, beta1, beta2, eps, wd, self._step_count)

    @staticmethod
    def _adamw_math(p, g, m, v, lr, beta1, beta2, eps, wd, step) -> None:
        p.mul_(1 - lr * wd)
        m.lerp_(g.to(m.dtype), 1 - beta1)
        v.mul_(beta2).addcmul_(g.to(v.dtype), g.to(v.dtype), value=1 - beta2)
        bc1, bc2 = 1 - beta1 ** step, 1 - beta2 ** step
        denom = (v.sqrt() / math.sqrt(bc2)).add_(eps)
        p.addcdiv_(m.to(p.dtype), denom.to(p.dtype), value=-lr / bc1)

    def _step_per_param(self) -> None:
        if self._clip:
            params = [p for g in self.param_groups for p in g["params"] if p.grad is not None]
            if params and self._norm_fn is not None:
                norm = self._norm_fn().float().sqrt()
                self.last_grad_norm = norm
                factor = torch.clamp(self._clip / (norm + 1e-6), max=1.0)
                for p in params:
                    p.grad.mul_(factor.to(p.grad.dtype))
            elif params:
                self.last_grad_norm = torch.nn.utils.clip_grad_norm_(params, self._clip)
        for group in self.param_groups:
            beta1, beta2 = group["betas"]
            for p in group["params"]:
                if p.grad is None:
                    continue
                st = self.state[p]
                if not st:
                    st["step"] = 0
                    st["exp_avg"] = torch.zeros_like(p, dtype=torch.float32)
                    st["exp_avg_sq"] = torch.zeros_like(p, dtype=torch.float32)
                st["step"] += 1
                self._adamw_math(p.data, p.grad.float(), st["exp_avg"], st["exp_avg_sq"], group["lr"], beta1, beta2,
                                 group["eps"], group["weight_decay"], st["step"])

    # -- checkpoint layout: per-parameter ``exp_avg / exp_avg_sq / step`` like torch AdamW ------
    def _owned_ranges(self, rank: Optional[int] = None):
        """``(global_offset, local_offset, n)`` pieces of the flat vector whose moments live on ``rank``."""
        if self._layout is not None:
            return self._layout(rank)
        if self._reducer is not None and hasattr(self._reducer, "owned_ranges"):
            return self._reducer.owned_ranges(rank)
        if self._shard is None:
            return [(0, 0, self._flat.numel)]
        n = self._shard[1]
        r = dist.get_rank() if rank is None else rank
        return [(r * n, 0, n)] if rank is not None else [(self._shard[0], 0, n)]

    def _full_moments(self) -> Tuple[torch.Tensor, torch.Tensor]:
        if self._shard is None or not dist.is_initialized():
            return self._m, self._v
        ws = dist.get_world_size()
        out = []
        for t in (self._m, self._v):
            pieces = [torch.empty_like(t) for _ in range(ws)]
            dist.all_gather(pieces, t)
            full = torch.zeros(self._flat.numel, dtype=t.dtype, device=t.device)
            for r in range(ws):
                for g, l, n in self._owned_ranges(r):
                    full[g:g + n] = pieces[r][l:l + n]
            out.append(full)
        return out[0], out[1]

    def state_dict(self) -> Dict[str, Any]:
        if self._flat is None:
            return super().state_dict()
        m, v = self._full_moments()
        state = {}
        for i, (p, off) in enumerate(zip(self._flat.params, self._flat.offsets)):
            state[i] = {"step": torch.tensor(float(self._step_count)),
                        "exp_avg": m[off:off + p.numel()].view(p.shape).detach().cpu().clone(),
                        "exp_avg_sq": v[off:off + p.numel()].view(p.shape).detach().cpu().clone()}
        group = {k: val for k, val in self.param_groups[0].items() if k != "params"}
        group["params"] = list(range(len(self._flat.params)))
        return {"state": state, "param_groups": [group]}

    def load_state_dict(self, state_dict: Dict[str, Any]) -> None:
        if self._flat is None:
            super().load_state_dict(state_dict)
            # torch casts loaded state to the parameter's dtype (bf16); the moments live in fp32, and a
            # resumed run has to continue with exactly the values that were saved
            params = [p for g in self.param_groups for p in g["params"]]
            keys = [i for g in state_dict["param_groups"] for i in g["params"]]
            for key, p in zip(keys, params):
                saved = state_dict["state"].get(key)
                if saved is None:
                    continue
                for name in ("exp_avg", "exp_avg_sq"):
                    if name in saved:
                        self.state[p][name] = saved[name].detach().to(device=p.device, dtype=torch.float32).clone()
            return
        for k, val in state_dict["param_groups"][0].items():
            if k != "params":
                self.param_groups[0][k] = val
        owned = self._owned_ranges()
        for i, (p, off) in enumerate(zip(self._flat.params, self._flat.offsets)):
            st = state_dict["state"].get(i) or state_dict["state"].get(str(i))
            if st is None:
                continue
            self._step_count = int(st["step"])
            for g, l, n in owned:
                lo, hi = max(off, g), min(off + p.numel(), g + n)
                if lo >= hi:
                    continue
                for name, dst in (("exp_avg", self._m), ("exp_avg_sq", self._v)):
                    src = st[name].reshape(-1)[lo - off:hi - off]
                    dst[l + lo - g:l + hi - g].copy_(src.to(dst.device, dst.dtype))


def newton_schulz_orthogonalize(G: torch.Tensor, steps: int = 5) -> torch.Tensor:
    """Quintic Newton-Schulz iteration pushing the singular values of ``G`` towards 1, times
    ``sqrt(max(1, rows / cols))``.

    The iteration runs on the unit-Frobenius-norm matrix (on its transpose when it is tall, so
    the Gram matrix is the small one) and the aspect-ratio factor is applied afterwards.  The
    reference multiplies by that factor *before* iterating (``astrai/trainer/optim.py:5-17``),
    which pushes low-rank tall matrices such as embedding gradients outside the convergence
    region of the polynomial and produces NaNs.
    """
    assert G.ndim == 2
    tall = G.size(0) > G.size(1)
    X = G.t() if tall else G
    X = X / (X.norm() + 1e-7)
    a, b, c = 3.4445, -4.7750, 2.0315
    for _ in range(steps):
        A = X @ X.t()
        X = a * X + (b * A + c * (A @ A)) @ X
    X = X.t() if tall else X
    return X * math.sqrt(max(1.0, G.size(0) / G.size(1)))


class Muon(Optimizer):
    def __init__(self, params, lr: float = 2e-3, momentum: float = 0.95, weight_decay: float = 0.0,
                 nesterov: bool = True, ns_steps: int = 5, adamw_lr: Optional[float] = None,
                 adamw_betas: Tuple[float, float] = (0.9, 0.95), adamw_eps: float = 1e-8, adamw_wd: float = 0.0):
        super().__init__(params, dict(lr=lr, momentum=momentum, weight_decay=weight_decay, nesterov=nesterov,
                                      ns_steps=ns_steps, adamw_lr=lr * 0.1 if adamw_lr is None else adamw_lr,
                                      adamw_betas=adamw_betas, adamw_eps=adamw_eps, adamw_wd=adamw_wd))

    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        for group in self.param_groups:
            for p in group["params"]:
                if p.grad is None:
                    continue
                if p.grad.is_sparse:
                    raise RuntimeError("Muon does not support sparse gradients")
                if p.ndim >= 2:
                    self._matrix_update(p, group)
                else:
                    self._vector_update(p, group)
        return loss

    def _matrix_update(self, p: torch.Tensor, group: Dict[str, Any]) -> None:
        lr, wd = group["lr"], group["weight_decay"]
        if wd:
            p.mul_(1 - lr * wd)
        grad = p.grad.add(p, alpha=wd) if group["nesterov"] else p.grad
        st = self.state[p]
        if "momentum_buffer" not in st:
            st["momentum_buffer"] = torch.zeros_like(grad)
        buf = st["momentum_buffer"].lerp_(grad, 1 - group["momentum"])
        shape = buf.shape
        update = newton_schulz_orthogonalize(buf.reshape(shape[0], -1), group["ns_steps"]).view(shape)
        p.add_(update, alpha=-lr * math.sqrt(max(1.0, p.size(0) / p.size(1))))

    def _vector_update(self, p: torch.Tensor, group: Dict[str, Any]) -> None:
        st = self.state[p]
        if not st:
            st["step"] = 0
            st["exp_avg"] = torch.zeros_like(p)
            st["exp_avg_sq"] = torch.zeros_like(p)
        st["step"] += 1
        beta1, beta2 = group["adamw_betas"]
        lr, wd = group["adamw_lr"], group["adamw_wd"]
        st["exp_avg"].lerp_(p.grad, 1 - beta1)
        st["exp_avg_sq"].lerp_(p.grad * p.grad, 1 - beta2)
        if wd:
            p.mul_(1 - lr * wd)
        denom = (st["exp_avg_sq"] / (1 - beta2 ** st["step"])).sqrt_().add_(group["adamw_eps"])
        p.addcdiv_(st["exp_avg"] / (1 - beta1 ** st["step"]), denom, value=-lr)
