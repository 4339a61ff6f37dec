"""Metric getters for the JSONL metric logger (reference: ``astrai/trainer/metric_util.py``).

Per-parameter gradient statistics are computed with one stacked device reduction per
statistic and a single device->host transfer, instead of one ``.item()`` per parameter.
"""

from __future__ import annotations

from typing import Callable, Dict

import torch
import torch.nn as nn


def _per_param(model: nn.Module, stat: Callable[[torch.Tensor], torch.Tensor], default) -> dict:
    names, values = [], []
    out = {}
    for name, p in model.named_parameters():
        out[name] = default
        if p.grad is not None:
            names.append(name)
            values.append(stat(p.grad.detach()).reshape(()).float())
    if values:
        for name, v in zip(names, torch.stack(values).tolist()):
            out[name] = v
    return out


def grad_norm(model: nn.Module, norm_type: int = 2) -> Dict[str, float]:
    return _per_param(model, lambda g: g.float().norm(norm_type), 0.0)


def grad_std(model: nn.Module) -> Dict[str, float]:
    return _per_param(model, lambda g: g.float().std(), 0.0)


def grad_max(model: nn.Module) -> Dict[str, float]:
    return _per_param(model, lambda g: g.max(), -float("inf"))


def grad_min(model: nn.Module) -> Dict[str, float]:
    return _per_param(model, lambda g: g.min(), float("inf"))


def grad_mean(model: nn.Module) -> Dict[str, float]:
    return _per_param(model, lambda g: g.float().mean(), 0.0)


def grad_nan_num(model: nn.Module) -> Dict[str, int]:
    return {k: int(v) for k, v in _per_param(model, lambda g: g.isnan().sum(), 0).items()}


METRICS: Dict[str, Callable] = {
    "loss": lambda ctx: ctx.loss,
    "lr": lambda ctx: ctx.optimizer.param_groups[-1]["lr"],
    "val_loss": lambda ctx: ctx.val_loss,
    "grad_norm": lambda ctx: grad_norm(ctx.model),
    "grad_std": lambda ctx: grad_std(ctx.model),
    "grad_max": lambda ctx: grad_max(ctx.model),
    "grad_min": lambda ctx: grad_min(ctx.model),
    "grad_mean": lambda ctx: grad_mean(ctx.model),
    "grad_nan_num": lambda ctx: grad_nan_num(ctx.model),
    "tokens_per_s": lambda ctx: ctx.kwargs.get("tokens_per_s", 0.0),   # set by the throughput callback
    "step_ms": lambda ctx: ctx.kwargs.get("step_ms", 0.0),
}
