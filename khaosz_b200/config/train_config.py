"""All knobs of a training run (reference: ``astrai/config/train_config.py:17-146``).

Adds, without renaming anything, the options the Blackwell executors understand:
``parallel_mode`` accepts ``"tp"`` besides ``none/ddp/fsdp`` and ``executor_kwargs`` may carry
``tp_size`` / ``fp8``.
"""

from __future__ import annotations

from dataclasses import dataclass, field, fields
from typing import Any, Callable, List, Optional

from .base import BaseConfig


def _opt(help: str, **meta):
    return {"help": help, **meta}


def _req(help: str):
    return {"help": help, "required": True}


@dataclass
class TrainConfig(BaseConfig):
    # -- what to train ------------------------------------------------------------------
    model_fn: Optional[Callable[[], Any]] = field(default=None, metadata=_req("Zero-argument model factory."))
    strategy: Optional[str] = field(default=None, metadata=_req("Training strategy: seq, sft, dpo or grpo."))
    dataset: Any = field(default=None, metadata=_req("Training dataset."))
    optimizer_fn: Optional[Callable[[Any], Any]] = field(default=None, metadata=_req("model -> optimizer."))
    scheduler_fn: Optional[Callable[[Any], Any]] = field(default=None, metadata=_req("optimizer -> LR scheduler."))
    n_epoch: int = field(default=1, metadata=_opt("Number of epochs."))
    batch_per_device: int = field(default=4, metadata=_opt("Micro-batch size per device."))
    grad_accum_steps: int = field(default=1, metadata=_opt("Micro-batches per optimizer step."))
    max_grad_norm: float = field(default=1.0, metadata=_opt("Global gradient-norm clip."))
    gradient_checkpointing_modules: list = field(
        default_factory=list, metadata=_opt("Module types whose forward is recomputed in backward."))
    # -- checkpoints --------------------------------------------------------------------
    start_epoch: int = field(default=0, metadata=_opt("Epoch to resume from."))
    start_batch: int = field(default=0, metadata=_opt("Batch iteration to resume from."))
    start_iteration: Optional[int] = field(default=None, metadata=_opt(
        "Value of the run-wide iteration counter to continue from (it runs across epochs); "
        "None: start_batch, as in the reference."))
    ckpt_dir: str = field(default="./checkpoint", metadata=_opt("Checkpoint directory."))
    ckpt_interval: int = field(default=5000, metadata=_opt("Iterations between checkpoints."))
    # -- LoRA ---------------------------------------------------------------------------
    lora: Any = field(default=None, metadata=_opt("LoRAConfig; None = full fine-tuning."))
    # -- metrics ------------------------------------------------------------------------
    log_dir: str = field(default="./checkpoint/logs", metadata=_opt("Directory of metric logs."))
    log_interval: int = field(default=100, metadata=_opt("Iterations between metric rows."))
    metrics: List[str] = field(default_factory=lambda: ["loss", "lr"], metadata=_opt("Metrics to record."))
    # -- data loading -------------------------------------------------------------------
    random_seed: int = field(default=3407, metadata=_opt("Sampler seed."))
    num_workers: int = field(default=0, metadata=_opt("DataLoader workers."))
    prefetch_factor: Optional[int] = field(default=None, metadata=_opt("DataLoader prefetch factor."))
    pin_memory: bool = field(default=False, metadata=_opt("Pin host batches."))
    # -- distributed --------------------------------------------------------------------
    nprocs: int = field(default=1, metadata=_opt("Processes (one per GPU)."))
    backend: str = field(default="nccl", metadata=_opt("torch.distributed backend."))
    master_addr: str = field(default="localhost", metadata=_opt("Rendezvous address."))
    master_port: str = field(default="29500", metadata=_opt("Rendezvous port."))
    parallel_mode: str = field(default="none", metadata=_opt("none, ddp, fsdp (fsdp_block where it applies, else fsdp_zero1), fsdp_block, fsdp_zero1, fsdp_full or tp."))
    start_method: str = field(default="spawn", metadata=_opt("Multiprocessing start method."))
    # -- misc ---------------------------------------------------------------------------
    device_type: str = field(default="cuda", metadata=_opt("Device type."))
    val_dataset: Any = field(default=None, metadata=_opt("Validation dataset."))
    val_split: Optional[float] = field(default=None, metadata=_opt("Fraction split off for validation."))
    val_step: int = field(default=1000, metadata=_opt("Optimizer steps between validations."))
    executor_kwargs: dict = field(default_factory=dict, metadata=_opt("Extra ExecutorFactory.create kwargs."))
    extra_kwargs: dict = field(default_factory=dict, metadata=_opt("Extra strategy kwargs."))

    def __post_init__(self):
        self.validate()

    def validate(self) -> None:
        missing = [f.name for f in fields(self) if f.metadata.get("required") and getattr(self, f.name) is None]
        if missing:
            raise ValueError(f"TrainConfig.{missing[0]} is required but got None.")
