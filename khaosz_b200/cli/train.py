"""Training CLI: ``python -m khaosz_b200.cli.train --train_type seq --param_path ... --data_root_path ...``.

Flag names and defaults are the reference's (``scripts/tools/train.py:15-190``); new here:
``--parallel_mode tp``, ``--tp_size``, ``--fp8`` and ``--optimizer {adamw,muon}``.  The model
is created in bf16, the optimizer is the fused flat AdamW and the schedule is warm-up +
cosine over the number of optimizer steps.
"""

from __future__ import annotations

import argparse
import logging
import os
from functools import partial

import torch

from ..config import AutoRegressiveLMConfig, TrainConfig
from ..data import DatasetFactory
from ..models import AutoRegressiveLM
from ..models.components.block import DecoderBlock
from ..models.components.lora import LoRAConfig
from ..parallel.fsdp_model import ShardedBlock
from ..parallel.tp_model import TPBlock
from ..serialization import find_latest_checkpoint
from ..trainer import CallbackFactory, FusedAdamW, Muon, SchedulerFactory, Trainer

log = logging.getLogger(__name__)


def parse_args(argv=None) -> argparse.Namespace:
    p = argparse.ArgumentParser(description="Train a decoder language model")
    p.add_argument("--train_type", choices=["seq", "sft", "dpo", "grpo"], required=True)
    p.add_argument("--data_root_path", type=str, required=True, help="Directory of token shards")
    p.add_argument("--param_path", type=str, required=True, help="Directory with config.json (and weights)")
    p.add_argument("--n_epoch", type=int, default=1)
    p.add_argument("--batch_per_device", type=int, default=1)
    p.add_argument("--grad_accum_steps", type=int, default=1)
    p.add_argument("--warmup_ratio", type=float, default=0.05)
    p.add_argument("--max_lr", type=float, default=3e-4)
    p.add_argument("--max_grad_norm", type=float, default=1.0)
    p.add_argument("--adamw_beta1", type=float, default=0.9)
    p.add_argument("--adamw_beta2", type=float, default=0.95)
    p.add_argument("--adamw_weight_decay", type=float, default=0.01)
    p.add_argument("--optimizer", choices=["adamw", "muon"], default="adamw")
    p.add_argument("--random_seed", type=int, default=3407)
    p.add_argument("--num_workers", type=int, default=4)
    p.add_argument("--no_pin_memory", dest="pin_memory", action="store_false", default=True)
    p.add_argument("--window_size", type=int, default=None, help="Tokens per sample (default: config.max_len)")
    p.add_argument("--stride", type=int, default=None)
    p.add_argument("--dpo_beta", type=float, default=0.1)
    p.add_argument("--group_size", type=int, default=4)
    p.add_argument("--grpo_clip_eps", type=float, default=0.2)
    p.add_argument("--grpo_kl_coef", type=float, default=0.01)
    p.add_argument("--grpo_sync_interval", type=int, default=200)
    p.add_argument("--label_smoothing", type=float, default=0.05)
    p.add_argument("--gradient_checkpointing", action="store_true", default=False)
    p.add_argument("--lora_r", type=int, default=0, help="Rank of the LoRA adapters (0 = train the full model).")
    p.add_argument("--lora_alpha", type=int, default=32)
    p.add_argument("--lora_target_modules", type=str, nargs="+", default=["q_proj", "v_proj"],
                   help="Names of the Linear layers that get adapters (q_proj k_proj v_proj o_proj gate up down).")
    p.add_argument("--ckpt_interval", type=int, default=5000)
    p.add_argument("--ckpt_dir", type=str, default="checkpoint")
    p.add_argument("--log_dir", type=str, default=None, help="Metric log directory (default: <ckpt_dir>/logs).")
    p.add_argument("--log_interval", type=int, default=10, help="Record the metrics every this many micro-batches.")
    p.add_argument("--metrics", type=str, nargs="+", default=["loss", "lr", "tokens_per_s", "step_ms"],
                   help="Metrics written to the JSONL log (see khaosz_b200.trainer.metrics.METRICS).")
    p.add_argument("--auto_resume", action="store_true", default=False,
                   help="Continue from the newest checkpoint under --ckpt_dir (weights, optimizer, scheduler and the "
                        "position in the data), if there is one; --param_path is used otherwise.")
    p.add_argument("--start_epoch", type=int, default=0)
    p.add_argument("--start_batch", type=int, default=0)
    p.add_argument("--master_addr", type=str, default="localhost")
    p.add_argument("--master_port", type=str, default="29500")
    p.add_argument("--backend", type=str, default="nccl")
    p.add_argument("--nprocs", type=int, default=1)
    p.add_argument("--parallel_mode", choices=["none", "ddp", "fsdp", "fsdp_block", "fsdp_zero1", "fsdp_full", "tp"], default="none")
    p.add_argument("--tp_size", type=int, default=None)
    p.add_argument("--cuda_graph", action="store_true", default=False,
                   help="replay forward+backward of a micro-batch as a CUDA graph (fixed batch shapes)")
    p.add_argument("--fp8", action="store_true", default=False, help="forward GEMMs of the linear layers in block-scaled fp8 (bf16 master weights)")
    p.add_argument("--device_type", type=str, default="cuda")
    p.add_argument("--start_method", type=str, default="spawn")
    return p.parse_args(argv)


def create_model(config: AutoRegressiveLMConfig):
    return AutoRegressiveLM(config).to(dtype=torch.bfloat16)


def create_optimizer(model, kind: str = "adamw", **kwargs):
    if kind == "muon":
        return Muon(model.parameters(), lr=kwargs["lr"], adamw_betas=kwargs["betas"], adamw_wd=kwargs["weight_decay"])
    return FusedAdamW(model.parameters(), **kwargs)


def compute_total_steps(dataset_len: int, n_epoch: int, batch_per_device: int, nprocs: int, grad_accum_steps: int) -> int:
    per_rank = -(-dataset_len // nprocs)
    batches = -(-per_rank // batch_per_device)
    return (batches // grad_accum_steps) * n_epoch


def train(args: argparse.Namespace) -> None:
    latest = find_latest_checkpoint(args.ckpt_dir) if getattr(args, "auto_resume", False) else None
    if latest is not None:
        args.param_path = latest[0]
    if not os.path.exists(args.param_path):
        raise FileNotFoundError(args.param_path)
    if args.nprocs > 1 and args.parallel_mode == "none":
        raise ValueError("--nprocs > 1 requires --parallel_mode to be 'ddp', 'fsdp', 'fsdp_block', 'fsdp_zero1', 'fsdp_full' or 'tp'")
    config = AutoRegressiveLMConfig.from_file(os.path.join(args.param_path, "config.json"))
    window = args.window_size or config.max_len
    dataset = DatasetFactory.load(train_type=args.train_type, load_path=args.data_root_path, window_size=window,
                                  stride=args.stride)
    # data-parallel replicas: the ranks of one tensor-parallel group read the same samples
    replicas = max(1, args.nprocs // (args.tp_size or args.nprocs)) if args.parallel_mode == "tp" else args.nprocs
    total = compute_total_steps(len(dataset), args.n_epoch, args.batch_per_device, replicas, args.grad_accum_steps)
    if latest is not None:
        # the iteration counter runs across epochs; the sampler wants the position inside the epoch
        per_epoch = -(-(-(-len(dataset) // replicas)) // args.batch_per_device)
        meta = latest[1]
        epoch = int(meta.get("epoch", 0))
        # continue after the last micro-batch whose gradient reached the weights (a periodic checkpoint is
        # taken before the optimizer step of its own iteration)
        iteration = int(meta.get("completed_iteration", meta.get("iteration", 0)))
        args.start_epoch = epoch
        args.start_batch = max(iteration - epoch * per_epoch, 0)
        args.start_iteration = iteration   # the counter keeps running across epochs and restarts
        log.info("resuming from %s (epoch %d, batch %d)", latest[0], args.start_epoch, args.start_batch)
    warmup = min(int(args.warmup_ratio * total), total)
    executor_kwargs = {"gradient_as_bucket_view": True, "broadcast_buffers": False}
    if args.fp8:
        executor_kwargs["fp8"] = True
    if args.cuda_graph:
        executor_kwargs["cuda_graph"] = True
    if args.parallel_mode == "tp":
        executor_kwargs["tp_size"] = args.tp_size or args.nprocs
    lora = None
    if args.lora_r > 0:
        if args.parallel_mode in ("tp", "fsdp_full", "fsdp_block"):
            raise ValueError("LoRA adapters train under --parallel_mode none, ddp or fsdp")
        lora = LoRAConfig(r=args.lora_r, alpha=args.lora_alpha, target_modules=tuple(args.lora_target_modules))
    cfg = TrainConfig(
        model_fn=partial(create_model, config), lora=lora, strategy=args.train_type, dataset=dataset,
        optimizer_fn=partial(create_optimizer, kind=args.optimizer, lr=args.max_lr,
                             betas=(args.adamw_beta1, args.adamw_beta2), weight_decay=args.adamw_weight_decay),
        scheduler_fn=partial(SchedulerFactory.create, schedule_type="cosine", warmup_steps=warmup,
                             lr_decay_steps=max(total - warmup, 1)),
        ckpt_dir=args.ckpt_dir, log_dir=args.log_dir or os.path.join(args.ckpt_dir, "logs"),
        log_interval=args.log_interval, metrics=args.metrics, n_epoch=args.n_epoch, batch_per_device=args.batch_per_device,
        start_epoch=args.start_epoch, start_batch=args.start_batch,
        start_iteration=getattr(args, "start_iteration", None), ckpt_interval=args.ckpt_interval,
        grad_accum_steps=args.grad_accum_steps, max_grad_norm=args.max_grad_norm, random_seed=args.random_seed,
        num_workers=args.num_workers, pin_memory=args.pin_memory, nprocs=args.nprocs, backend=args.backend,
        master_addr=args.master_addr, master_port=args.master_port, parallel_mode=args.parallel_mode,
        device_type=args.device_type, start_method=args.start_method,
        gradient_checkpointing_modules=[DecoderBlock, TPBlock, ShardedBlock] if args.gradient_checkpointing else [],
        executor_kwargs=executor_kwargs,
        extra_kwargs={"beta": args.dpo_beta, "label_smoothing": args.label_smoothing, "clip_eps": args.grpo_clip_eps,
                      "kl_coef": args.grpo_kl_coef, "group_size": args.group_size,
                      "sync_interval": args.grpo_sync_interval})
    callbacks = []
    if lora is not None:   # the adapters alone, beside the full checkpoints
        callbacks.append(CallbackFactory.create("lora_adapter", os.path.join(args.ckpt_dir, "lora_adapter"), lora))
    Trainer(cfg, callbacks=callbacks).train(resume_dir=args.param_path)


if __name__ == "__main__":
    train(parse_args())
