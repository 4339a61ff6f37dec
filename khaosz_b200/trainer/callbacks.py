"""Trainer callbacks: gradient clipping, activation checkpointing, checkpoints, progress bar,
JSONL metric log and validation (reference: ``astrai/trainer/train_callback.py:36-333``).

Hooks (all optional): ``on_train_begin/end``, ``on_epoch_begin/end``, ``on_batch_begin/end``,
``on_optimizer_step``, ``on_error``; each receives the ``TrainContext``.
"""

from __future__ import annotations

import json
import logging
import os
import sys
import time
from pathlib import Path
from typing import IO, Callable, List, Optional, Protocol, runtime_checkable

import torch
import torch.distributed as dist
import torch.nn as nn
from torch.nn.utils import clip_grad_norm_
from torch.utils.checkpoint import checkpoint as recompute
from tqdm import tqdm

from ..factory import BaseFactory
from ..parallel.setup import get_current_device, get_rank, only_on_rank
from ..serialization import Checkpoint
from .metrics import METRICS

log = logging.getLogger(__name__)


@runtime_checkable
class TrainCallback(Protocol):
    def on_train_begin(self, context): ...
    def on_train_end(self, context): ...
    def on_epoch_begin(self, context): ...
    def on_epoch_end(self, context): ...
    def on_batch_begin(self, context): ...
    def on_batch_end(self, context): ...
    def on_optimizer_step(self, context): ...
    def on_error(self, context): ...


class CallbackFactory(BaseFactory[TrainCallback]):
    pass


@CallbackFactory.register("gradient_clipping")
class GradientClippingCallback:
    """Global-norm clipping.  With a ``FusedAdamW`` optimizer the norm and the clip factor are
    computed on the device inside the optimizer step (correct across FSDP shards, no host
    sync); any other optimizer gets ``clip_grad_norm_``."""

    def __init__(self, max_grad_norm: float):
        self.max_grad_norm = max_grad_norm

    def on_optimizer_step(self, context):
        fused = getattr(context.optimizer, "fused_clip", None)
        if callable(fused):
            fused(self.max_grad_norm)
        elif self.max_grad_norm and self.max_grad_norm > 0:
            clip_grad_norm_(context.model.parameters(), self.max_grad_norm)


@CallbackFactory.register("device_health")
class DeviceHealthCallback:
    """Turns a device-side failure into a Python exception.

    Every wait inside the kernels is bounded; a wait that runs out (a peer rank that never
    arrives, a copy that never completes) records a code in a per-device error word and the kernel
    returns instead of hanging.  The word is read

    * before every optimizer step (one 4-byte synchronising copy per accumulation window), so that
      gradients of a failed forward / backward never reach the weights;
    * after every optimizer step through a non-blocking probe (an asynchronous copy plus an event
      that the next batches poll), so that a failure inside the fused reduce + update kernels -
      which refuse to touch moments and parameters once the word is set - surfaces within a batch
      or two and not a whole accumulation window later;
    * at the end of training, so that a failure in the last step is not lost.

    The raised ``KernelError`` takes the trainer's error path; the checkpoint callback then writes
    no resumable checkpoint (the ranks may disagree about what was applied)."""

    def __init__(self, check=None, probe=None):
        self._check = check
        self._probe = probe
        self._step_pending = False

    def _ready(self) -> bool:
        if self._check is None:
            if not torch.cuda.is_available():
                return False
            from ..ops import raise_on_device_error
            from ..ops._lib import ErrorProbe

            self._check = raise_on_device_error
            if self._probe is None:
                self._probe = ErrorProbe()
        return True

    def on_optimizer_step(self, context):
        if self._ready():
            self._check()
            self._step_pending = True

    def on_batch_begin(self, context):
        if self._probe is not None:
            if self._step_pending:       # the optimizer step of the previous batch has been enqueued
                self._step_pending = False
                self._probe.post()
            self._probe.poll()

    def on_train_end(self, context):
        if context.kwargs.get("error") is not None or not self._ready():
            return
        self._check()


_TOKEN_KEYS = ("input_ids", "chosen", "rejected", "prompts", "responses")


def batch_tokens(batch) -> int:
    """Tokens in one micro-batch of any of the dataset layouts (seq / sft / dpo / grpo)."""
    if torch.is_tensor(batch):
        return batch.numel()
    if isinstance(batch, dict):
        return sum(v.numel() for k, v in batch.items() if k in _TOKEN_KEYS and torch.is_tensor(v))
    return 0


@CallbackFactory.register("throughput")
class ThroughputCallback:
    """Step time and whole-job tokens per second, published as ``context.kwargs["step_ms"]`` and
    ``context.kwargs["tokens_per_s"]`` (the ``step_ms`` / ``tokens_per_s`` metrics read them).

    On a GPU the step is timed on the device: one CUDA event per optimizer step on the current
    stream, and the interval between two consecutive events is read once both have completed
    (``Event.query``), so the host never waits for the device; the published figure therefore lags
    the running step by one or two steps.  On CPU the host clock is used.  The reference records
    no throughput (``astrai/trainer/metric_util.py:18-75`` has loss, lr and gradient statistics only)."""

    def __init__(self, clock: Callable[[], float] = time.perf_counter, use_cuda: Optional[bool] = None):
        self._clock = clock
        self._use_cuda = use_cuda
        self._tokens = 0
        self._marks: List[tuple] = []    # (event or host time, tokens since the previous mark)

    def on_batch_end(self, context):
        self._tokens += context.kwargs.get("batch_tokens", 0)

    def _replicas(self, context) -> int:
        sampler = getattr(context.dataloader, "sampler", None)
        return int(getattr(sampler, "num_replicas", None) or context.world_size or 1)

    def _publish(self, context, seconds: float, tokens: int) -> None:
        if seconds > 0:
            context.kwargs["step_ms"] = seconds * 1e3
            context.kwargs["tokens_per_s"] = tokens * self._replicas(context) / seconds

    def on_optimizer_step(self, context):
        if self._use_cuda is None:
            self._use_cuda = torch.cuda.is_available() and torch.device(get_current_device()).type == "cuda"
        tokens, self._tokens = self._tokens, 0
        if not self._use_cuda:
            now = self._clock()
            if self._marks:
                self._publish(context, now - self._marks[-1][0], tokens)
            self._marks = [(now, tokens)]
            return
        event = torch.cuda.Event(enable_timing=True)
        event.record()
        self._marks.append((event, tokens))
        # the newest pair of consecutive marks that the device has already passed
        done = [i for i, (ev, _) in enumerate(self._marks) if ev.query()]
        if len(done) >= 2:
            last = done[-1]
            self._publish(context, self._marks[last - 1][0].elapsed_time(self._marks[last][0]) * 1e-3,
                          self._marks[last][1])
            self._marks = self._marks[last:]
        elif len(self._marks) > 64:          # a device that never catches up: do not grow without bound
            self._marks = self._marks[-2:]


@CallbackFactory.register("gradient_checkpointing")
class GradientCheckpointingCallback:
    """Recompute the forward of the listed module types during backward."""

    def __init__(self, modules: Optional[List[type]] = None):
        self.modules = tuple(modules) if modules else ()

    def _enable(self, module: nn.Module) -> None:
        if self.modules and isinstance(module, self.modules) and not hasattr(module, "_original_forward"):
            inner = module.forward
            module._original_forward = inner
            module.forward = lambda *a, **kw: recompute(inner, *a, use_reentrant=False, **kw)

    @staticmethod
    def _disable(module: nn.Module) -> None:
        inner = getattr(module, "_original_forward", None)
        if inner is not None:
            module.forward = inner
            del module._original_forward

    def on_train_begin(self, context):
        context.model.apply(self._enable)

    def on_train_end(self, context):
        context.model.apply(self._disable)


@CallbackFactory.register("checkpoint")
class CheckpointCallback:
    extra_keys = ("optimizer", "scheduler")

    def __init__(self, save_dir: str, interval: int, weight_only: bool = False,
                 save_extra_fn: Optional[Callable] = None):
        self.save_dir, self.interval, self.weight_only = save_dir, interval, weight_only
        self.save_extra_fn = save_extra_fn or self.save_extra
        self.last_ckpt_iter = 0

    @staticmethod
    def save_extra(context) -> dict:
        return {name: getattr(context, name).state_dict() for name in CheckpointCallback.extra_keys
                if getattr(context, name, None)}

    def _save(self, context) -> None:
        state = context.executor.unwrap_model(context.model)  # collective under sharded executors
        extra = {} if self.weight_only else self.save_extra_fn(context)  # may gather optimizer shards
        self.last_ckpt_iter = context.iteration
        # micro-batches whose gradients are already in the weights: a periodic checkpoint is taken before the
        # optimizer step of its own iteration, so a run that continues from it has to start from here
        applied = (context.kwargs.get("start_iteration", 0)
                   + context.kwargs.get("optimizer_steps", 0) * context.executor.grad_accum_steps)
        if get_rank() == 0:
            path = os.path.join(self.save_dir, f"epoch_{context.epoch}_iter_{context.iteration}")
            context.checkpoint = Checkpoint(state_dict=state, epoch=context.epoch, iteration=context.iteration,
                                            extra=extra, config=context.model_config,
                                            meta={"completed_iteration": min(applied, context.iteration)})
            context.checkpoint.save(path)

    def on_train_begin(self, context):
        # a resumed run counts its interval from where it continues, not from zero
        self.last_ckpt_iter = context.iteration

    def on_batch_end(self, context):
        if context.iteration - self.last_ckpt_iter >= self.interval:
            self._save(context)

    def on_train_end(self, context):
        if context.iteration != self.last_ckpt_iter:
            self._save(context)

    def on_error(self, context):
        from ..ops._lib import KernelError

        if isinstance(context.kwargs.get("error"), KernelError):
            # a device-side failure (a collective that gave up): the ranks may hold different weights,
            # and an automatic resume must not pick such a state up
            log.error("device-side failure: no emergency checkpoint is written; resume from the last periodic one")
            return
        self._save(context)


@CallbackFactory.register("lora_adapter")
class LoRAAdapterCallback:
    """Writes the adapters of a LoRA run (``adapter_model.safetensors`` + ``adapter_config.json``,
    the layout of ``astrai/model/components/lora.py:121-137``) to ``save_dir`` when training ends -
    after an error too, since ``on_train_end`` always runs."""

    def __init__(self, save_dir: str, config):
        self.save_dir, self.config = save_dir, config

    def _save(self, context) -> None:
        from ..models.components.lora import save_lora

        if get_rank() == 0:
            save_lora(context.model, self.save_dir, self.config)

    def on_train_end(self, context):
        self._save(context)


@CallbackFactory.register("progress_bar")
class ProgressBarCallback:
    def __init__(self, num_epoch: int, log_interval: int = 100, file: Optional[IO[str]] = None):
        self.num_epoch, self.log_interval, self.file = num_epoch, max(int(log_interval), 1), file
        self.progress_bar: Optional[tqdm] = None

    @only_on_rank(0)
    def on_epoch_begin(self, context):
        self.progress_bar = tqdm(total=len(context.dataloader), desc=f"Epoch {context.epoch + 1}/{self.num_epoch}",
                                 dynamic_ncols=True, file=self.file or sys.stdout)

    @only_on_rank(0)
    def on_batch_end(self, context):
        if self.progress_bar is None:
            return
        # reading the loss waits for the device; do it at the logging cadence only on GPUs
        if not torch.cuda.is_available() or context.iteration % self.log_interval == 0:
            postfix = {"loss": f"{context.loss:.4f}", "lr": f"{context.optimizer.param_groups[-1]['lr']:.2e}"}
            if context.val_loss > 0:
                postfix["val_loss"] = f"{context.val_loss:.4f}"
            if context.kwargs.get("tokens_per_s"):       # published by the throughput callback
                postfix["tok/s"] = f"{context.kwargs['tokens_per_s']:,.0f}"
            self.progress_bar.set_postfix(postfix, refresh=False)
        self.progress_bar.update(1)

    @only_on_rank(0)
    def on_epoch_end(self, context):
        if self.progress_bar is not None:
            self.progress_bar.close()
            self.progress_bar = None


@CallbackFactory.register("metric_logger")
class MetricLoggerCallback:
    """Rows ``{timestamp, epoch, iter, <metrics>}`` written to
    ``<log_dir>/epoch_E_iter_I_metric.jsonl`` every ``save_interval`` iterations, at the end
    and on error."""

    def __init__(self, log_dir: str, save_interval: int, log_interval: int = 10, metrics: List[str] = None):
        self.save_interval, self.log_interval = save_interval, max(int(log_interval), 1)
        self.metrics = list(metrics) if metrics else ["loss", "lr"]
        self.log_dir = Path(log_dir) if log_dir else Path.cwd() / "logs"
        self.log_dir.mkdir(parents=True, exist_ok=True)
        self.rows: List[dict] = []
        self.last_log_iter = 0
        unknown = [m for m in self.metrics if m not in METRICS]
        if unknown:
            raise ValueError(f"Unknown metrics: {unknown}; available: {sorted(METRICS)}")

    def _row(self, context) -> dict:
        row = {"timestamp": time.strftime("%Y-%m-%dT%H:%M:%S"), "epoch": context.epoch, "iter": context.iteration}
        row.update({m: METRICS[m](context) for m in self.metrics})
        return row

    def _flush(self, context) -> None:
        self.last_log_iter = context.iteration
        if get_rank() != 0:
            return
        path = self.log_dir / f"epoch_{context.epoch}_iter_{context.iteration}_metric.jsonl"
        with open(path, "w") as fh:
            fh.writelines(json.dumps(r) + "\n" for r in self.rows)

    def on_batch_end(self, context):
        if context.iteration % self.log_interval == 0 and get_rank() == 0:
            self.rows.append(self._row(context))
        if context.iteration - self.last_log_iter >= self.save_interval:
            self._flush(context)

    def on_train_end(self, context):
        if context.iteration != self.last_log_iter:
            self._flush(context)

    def on_error(self, context):
        self._flush(context)


@CallbackFactory.register("validation")
class ValidationCallback:
    """Mean strategy loss over the validation loader every ``val_step`` optimizer steps,
    averaged over ranks."""

    def _validate(self, context) -> None:
        context.model.eval()
        total, batches = None, 0
        with torch.no_grad():
            for batch in context.val_dataloader:
                loss = context.strategy(batch).detach().float()
                total = loss if total is None else total + loss
                batches += 1
        mean = (total / max(batches, 1)) if total is not None else torch.zeros(())
        if context.world_size > 1 and dist.is_initialized():
            mean = mean.to(get_current_device()) if dist.get_backend() == "nccl" else mean.cpu()
            dist.all_reduce(mean)
            mean = mean / context.world_size
        context.val_loss = float(mean)
        context.model.train()
        log.info("Epoch %d, Step %d, Val Loss: %.4f", context.epoch + 1,
                 context.iteration // context.config.grad_accum_steps, context.val_loss)

    def on_optimizer_step(self, context):
        cfg = context.config
        if context.val_dataloader is None or cfg.val_step <= 0:
            return
        if (context.iteration // cfg.grad_accum_steps) % cfg.val_step == 0:
            self._validate(context)
