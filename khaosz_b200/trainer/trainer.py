"""The training loop (reference: ``astrai/trainer/trainer.py:15-109``).

Default callbacks, in order: gradient_checkpointing, checkpoint, metric_logger, progress_bar,
gradient_clipping, validation, device_health, throughput; user callbacks run after them.  Any
exception triggers the ``on_error`` hooks (emergency checkpoint, metric flush) and is re-raised;
``on_train_end`` always runs.
"""

from __future__ import annotations

import logging
from typing import List, Optional

from ..config.train_config import TrainConfig
from ..parallel.setup import spawn_parallel_fn
from ..utils.trace import trace_range
from .callbacks import CallbackFactory, TrainCallback, batch_tokens
from .context import TrainContext, TrainContextBuilder

log = logging.getLogger(__name__)


class Trainer:
    def __init__(self, train_config: TrainConfig, callbacks: Optional[List[TrainCallback]] = None):
        self.train_config = train_config
        self.callbacks: List[TrainCallback] = self._get_default_callbacks() + list(callbacks or [])

    def _get_default_callbacks(self) -> List[TrainCallback]:
        cfg = self.train_config
        make = CallbackFactory.create
        return [
            make("gradient_checkpointing", modules=cfg.gradient_checkpointing_modules),
            make("checkpoint", cfg.ckpt_dir, cfg.ckpt_interval),
            make("metric_logger", log_dir=cfg.log_dir, save_interval=cfg.ckpt_interval,
                 log_interval=cfg.log_interval, metrics=cfg.metrics),
            make("progress_bar", cfg.n_epoch, log_interval=cfg.log_interval),
            make("gradient_clipping", cfg.max_grad_norm),
            make("validation"),
            make("device_health"),
            make("throughput"),
        ]

    def _call_callbacks(self, hook: str, context: TrainContext) -> None:
        for cb in self.callbacks:
            fn = getattr(cb, hook, None)
            if fn is not None:
                fn(context)

    def _micro_step(self, context: TrainContext, batch) -> None:
        executor = context.executor
        context.kwargs["batch_tokens"] = batch_tokens(batch)
        with executor.accumulate(context.model):
            if hasattr(executor, "micro_step"):   # forward + backward, optionally as a replayed CUDA graph
                with trace_range("micro_step"):
                    context.loss = executor.micro_step(context.strategy, batch)
            else:
                loss = context.strategy(batch)
                context.loss = loss.detach()
                executor.backward(loss / executor.grad_accum_steps)
            context.iteration += 1
            self._call_callbacks("on_batch_end", context)
            if executor.sync_gradients:
                self._call_callbacks("on_optimizer_step", context)
                with trace_range("optimizer_step"):
                    context.optimizer.step()
                    context.optimizer.zero_grad()
                context.kwargs["optimizer_steps"] = context.kwargs.get("optimizer_steps", 0) + 1
                if context.scheduler:
                    context.scheduler.step()

    def _trainer_loop(self, resume_dir: Optional[str] = None) -> None:
        context = TrainContextBuilder(self.train_config).with_resume_dir(resume_dir).build()
        context.kwargs["start_iteration"] = context.iteration
        self._call_callbacks("on_train_begin", context)
        try:
            context.model.train()
            for epoch in range(context.epoch, context.config.n_epoch):
                context.epoch = epoch
                self._call_callbacks("on_epoch_begin", context)
                for batch in context.dataloader:
                    self._call_callbacks("on_batch_begin", context)
                    self._micro_step(context, batch)
                self._call_callbacks("on_epoch_end", context)
        except Exception as exc:
            log.error("Training failed: %s", exc, exc_info=True)
            context.kwargs["error"] = exc
            self._call_callbacks("on_error", context)
            raise
        finally:
            self._call_callbacks("on_train_end", context)

    def train(self, resume_dir: Optional[str] = None) -> None:
        cfg = self.train_config
        spawn_parallel_fn(self._trainer_loop, world_size=cfg.nprocs, backend=cfg.backend,
                          master_addr=cfg.master_addr, master_port=cfg.master_port, device_type=cfg.device_type,
                          start_method=cfg.start_method, resume_dir=resume_dir)
