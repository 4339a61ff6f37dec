"""Mutable state of one training run and the builder that assembles it.

Build order follows ``astrai/trainer/train_context.py:54-183``: executor -> model on the
rank's device -> resume weights -> LoRA -> optimizer / scheduler -> validation split ->
sampler + DataLoader -> ``executor.prepare`` -> optimizer / scheduler state -> strategy.

The loss of a micro-batch reaches the host through a pinned buffer and an event instead of a
blocking ``.item()``; ``context.loss`` waits for that copy only when somebody reads it.
"""

from __future__ import annotations

import logging
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any, Optional

import torch
import torch.nn as nn
from torch.utils.data import DataLoader, random_split

from ..config.train_config import TrainConfig
from ..data.sampler import ResumableDistributedSampler
from ..models.components.lora import inject_lora
from ..parallel.executor import BaseExecutor, ExecutorFactory
from ..parallel.setup import get_current_device, get_rank, get_world_size
from ..serialization import CONFIG_FILE, META_FILE, Checkpoint, load_json, load_model_weights
from .strategy import BaseStrategy, StrategyFactory

log = logging.getLogger(__name__)


class _AsyncScalar:
    """Device scalar -> pinned host memory without stalling the launching thread."""

    def __init__(self) -> None:
        self._host: Optional[torch.Tensor] = None
        self._event = None
        self._value = 0.0

    def set(self, value) -> None:
        if torch.is_tensor(value) and value.is_cuda:
            if self._host is None:
                self._host = torch.zeros(1, dtype=torch.float32).pin_memory()
                self._event = torch.cuda.Event()
            self._host.copy_(value.detach().reshape(1).float(), non_blocking=True)
            self._event.record()
            self._pending = True
        else:
            self._value = float(value)
            self._pending = False

    _pending = False

    def get(self) -> float:
        if self._pending:
            self._event.synchronize()
            self._value = float(self._host[0])
            self._pending = False
        return self._value


@dataclass
class TrainContext:
    model: nn.Module = None
    strategy: BaseStrategy = None
    dataloader: DataLoader = None
    optimizer: Any = None
    scheduler: Any = None
    checkpoint: Checkpoint = None
    config: TrainConfig = None
    model_config: dict = field(default_factory=dict)
    executor: BaseExecutor = None
    epoch: int = 0
    iteration: int = 0
    val_dataloader: DataLoader = None
    val_loss: float = 0.0
    world_size: int = 1
    rank: int = 0
    kwargs: dict = field(default_factory=dict)
    _loss: _AsyncScalar = field(default_factory=_AsyncScalar, repr=False)

    @property
    def loss(self) -> float:
        return self._loss.get()

    @loss.setter
    def loss(self, value) -> None:
        self._loss.set(value)


def _loader(dataset, sampler, cfg: TrainConfig) -> DataLoader:
    return DataLoader(dataset, batch_size=cfg.batch_per_device, sampler=sampler, num_workers=cfg.num_workers,
                      pin_memory=cfg.pin_memory and torch.cuda.is_available(), prefetch_factor=cfg.prefetch_factor)


class TrainContextBuilder:
    def __init__(self, config: TrainConfig):
        self.config = config
        self._resume_dir: Optional[str] = None

    def with_resume_dir(self, resume_dir: Optional[str]) -> "TrainContextBuilder":
        self._resume_dir = resume_dir
        return self

    def _resume(self, ctx: TrainContext, model: nn.Module) -> None:
        root = Path(self._resume_dir)
        if (root / META_FILE).exists():
            ckpt = Checkpoint.load(str(root))
            if ckpt.config:
                ctx.model_config = ckpt.config
            model.load_state_dict(ckpt.state_dict, strict=False)
            # the position comes from the config (CLI flags), as in the reference: start_batch is the
            # position inside start_epoch (what the sampler skips); the iteration counter itself runs
            # across epochs, so a resumed run continues it from start_iteration when that is given
            ctx.epoch = self.config.start_epoch
            ctx.iteration = self.config.start_batch if self.config.start_iteration is None else self.config.start_iteration
            ctx.kwargs["epoch_start_batch"] = self.config.start_batch
            ctx.checkpoint = ckpt
        elif any(root.glob("*.safetensors")):
            model.load_state_dict(load_model_weights(str(root)), strict=False)
        else:  # a parameter directory with only config.json: train from the random initialisation
            log.info("no weights in %s: starting from the random initialisation", root)

    def build(self) -> TrainContext:
        cfg = self.config
        device = get_current_device()
        executor = ExecutorFactory.create(cfg.parallel_mode, grad_accum_steps=cfg.grad_accum_steps,
                                          **cfg.executor_kwargs)
        model = cfg.model_fn().to(device=device)
        model_config = {}
        if self._resume_dir and (Path(self._resume_dir) / CONFIG_FILE).exists():
            model_config = load_json(Path(self._resume_dir) / CONFIG_FILE)
        if not model_config and hasattr(model, "config") and hasattr(model.config, "to_dict"):
            model_config = model.config.to_dict()
        ctx = TrainContext(model=model, world_size=get_world_size(), rank=get_rank(), config=cfg,
                           model_config=model_config, executor=executor)
        if self._resume_dir is not None:
            self._resume(ctx, model)
        if cfg.lora is not None:
            inject_lora(model, r=cfg.lora.r, alpha=cfg.lora.alpha, target_modules=set(cfg.lora.target_modules))
            if ctx.checkpoint is not None:
                # the adapters did not exist yet when the checkpoint's weights were loaded above
                adapters = {k: v for k, v in ctx.checkpoint.state_dict.items() if k.rpartition(".")[2] in ("lora_A", "lora_B")}
                if adapters:
                    model.load_state_dict(adapters, strict=False)
        ctx.optimizer = cfg.optimizer_fn(model)
        ctx.scheduler = cfg.scheduler_fn(ctx.optimizer)

        train_set, val_set = cfg.dataset, cfg.val_dataset
        if val_set is None and cfg.val_split is not None:
            n_val = max(1, int(len(cfg.dataset) * cfg.val_split))
            gen = torch.Generator().manual_seed(cfg.random_seed)
            train_set, val_set = random_split(cfg.dataset, [len(cfg.dataset) - n_val, n_val], generator=gen)
        sampler = ResumableDistributedSampler(train_set, start_epoch=ctx.epoch,
                                              start_iter=ctx.kwargs.get("epoch_start_batch", 0) * cfg.batch_per_device,
                                              seed=cfg.random_seed)
        ctx.dataloader = _loader(train_set, sampler, cfg)
        if val_set is not None:
            val_sampler = ResumableDistributedSampler(val_set, seed=cfg.random_seed, shuffle=False)
            ctx.val_dataloader = _loader(val_set, val_sampler, cfg)

        ctx.model, ctx.optimizer, ctx.dataloader, ctx.scheduler = executor.prepare(
            model, ctx.optimizer, ctx.dataloader, ctx.scheduler)
        if ctx.checkpoint is not None and ctx.checkpoint.extra:
            for name in ("optimizer", "scheduler"):
                target = getattr(ctx, name, None)
                if target is not None and name in ctx.checkpoint.extra:
                    target.load_state_dict(ctx.checkpoint.extra[name])
        ctx.strategy = StrategyFactory.create(cfg.strategy, ctx.model, device, executor=executor,
                                              model_fn=cfg.model_fn, **cfg.extra_kwargs)
        return ctx
