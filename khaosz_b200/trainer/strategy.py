"""Loss strategies: ``seq`` (next token), ``sft`` (masked), ``dpo`` and ``grpo``.

Same objectives as ``astrai/trainer/strategy.py:100-334``.  The logits never get an fp32
copy: the label-smoothed cross entropy and the per-token log-probabilities come from the
fused kernels in ``khaosz_b200.ops`` (which fall back to the PyTorch formulas on CPU).

GRPO batch layout (the reference leaves it inconsistent between dataset and strategy):
``prompts [B, P]``, ``responses [B, G, R]``, ``masks [B, G, R]``, ``rewards [B, G]``.  Flat
windows from ``GRPODataset`` (``responses [B, G*R]``, ``rewards [B, G*R]``) are folded into
that layout with ``group_size``; a group's reward is the mean over its window.
"""

from __future__ import annotations

from abc import ABC, abstractmethod
from typing import Callable, Dict

import torch
import torch.nn as nn
import torch.nn.functional as F
from torch import Tensor

from .. import ops
from ..factory import BaseFactory

IGNORE_INDEX = -100


def move_to_device(batch: Dict[str, Tensor], device) -> Dict[str, Tensor]:
    return {k: v.to(device, non_blocking=True) if torch.is_tensor(v) else v for k, v in batch.items()}


def create_ref_model(model_fn: Callable[[], nn.Module], state_dict: dict, like: nn.Module = None,
                     shard_like=None) -> nn.Module:
    """Frozen copy of the policy built from ``model_fn`` and a full state dict.  When the policy is
    sliced (tensor parallel) or sharded (fully sharded) the copy is cut the same way, so it costs
    ``1 / world`` of the memory and runs through the same fused GEMM + collective kernels.
    ``shard_like``: the ``ShardedUnits`` of a policy that is sharded block by block; the copy's blocks are
    then sharded over the same group and gathered block by block when it is evaluated."""
    ref = model_fn()
    if like is not None:
        p = next(like.parameters())
        ref = ref.to(device=p.device, dtype=p.dtype)
    ref.load_state_dict(state_dict)
    if like is not None and hasattr(like, "info"):
        from ..parallel.fsdp_model import FullShardLM, full_shard
        from ..parallel.tp_model import TensorParallelLM, tensorize

        if isinstance(like, TensorParallelLM):
            ref = tensorize(ref, like.info.group)
        elif isinstance(like, FullShardLM):
            ref = full_shard(ref, like.info.group)
    ref.requires_grad_(False)
    ref.eval()
    if shard_like is not None:
        from ..parallel.unit_shard import ShardedUnits

        ref.sharded_units = ShardedUnits(ref, group=shard_like.group, prefetch=shard_like.prefetch, frozen=True)
        return ref
    if like is not None and next(ref.parameters()).is_cuda and hasattr(ref, "pack_parameters"):
        ref.pack_parameters(with_grad=False)
    return ref


def get_logprobs(model, input_ids: Tensor, mask: Tensor, reduction: str) -> Tensor:
    """Masked log-probabilities of ``input_ids[:, 1:]`` under ``model``; ``reduction`` over the
    sequence is ``mean`` | ``sum`` | ``none``."""
    if reduction not in ("mean", "sum", "none"):
        raise ValueError(f"reduction must be one of ['mean', 'sum', 'none'], got '{reduction}'")
    targets, m = input_ids[:, 1:], mask[:, 1:].to(torch.float32)
    logits = model(input_ids[:, :-1].contiguous(), mask[:, :-1])["logits"]
    if hasattr(model, "gather_tokens"):  # tensor parallel: logits of this rank's token slice only
        local = ops.token_logprobs(logits, model.shard_targets(targets.contiguous()))
        lp = model.gather_tokens(local, targets.shape) * m
    else:
        lp = ops.token_logprobs(logits, targets.contiguous()) * m
    if reduction == "none":
        return lp
    total = lp.sum(dim=-1)
    return total / m.sum(dim=-1).clamp(min=1.0) if reduction == "mean" else total


def local_loss(model, logits: Tensor, targets: Tensor, label_smoothing: float) -> Tensor:
    """Mean label-smoothed cross entropy.  A tensor-parallel model returns the logits of its
    token slice only: the targets are cut to that slice and the local mean is weighted so that
    the ranks' losses add up to the global mean."""
    shard = getattr(model, "shard_targets", None)
    if shard is None:
        return ops.cross_entropy(logits, targets, label_smoothing, IGNORE_INDEX)
    local = shard(targets)
    return ops.cross_entropy(logits, local, label_smoothing, IGNORE_INDEX) * model.loss_weight(local, IGNORE_INDEX, targets)


class BaseStrategy(ABC):
    def __init__(self, model, device, **kwargs):
        self.model, self.device = model, device
        self.executor = kwargs.pop("executor", None)
        self.model_fn = kwargs.pop("model_fn", None)
        self.extra_kwargs = kwargs

    @abstractmethod
    def compute_loss(self, batch: Dict[str, Tensor]) -> Tensor: ...

    def __call__(self, batch: Dict[str, Tensor]) -> Tensor:
        return self.compute_loss(batch)

    def _make_ref(self) -> nn.Module:
        state = self.executor.unwrap_model(self.model) if self.executor is not None else self.model.state_dict()
        return create_ref_model(self.model_fn, state, like=self.model,
                                shard_like=getattr(self.executor, "units", None))


class StrategyFactory(BaseFactory[BaseStrategy]):
    @classmethod
    def _validate_component(cls, strategy_cls: type) -> None:
        if not (isinstance(strategy_cls, type) and issubclass(strategy_cls, BaseStrategy)):
            raise TypeError(f"{getattr(strategy_cls, '__name__', strategy_cls)} must inherit from BaseStrategy")

    @classmethod
    def create(cls, train_type: str, model, device, **kwargs) -> BaseStrategy:
        return super().create(train_type, model, device, **kwargs)

    @classmethod
    def available_strategies(cls) -> list:
        return cls.list_registered()


@StrategyFactory.register("seq")
class SEQStrategy(BaseStrategy):
    def __init__(self, model, device, label_smoothing: float = 0.0, **kwargs):
        super().__init__(model, device, **kwargs)
        self.label_smoothing = label_smoothing

    def compute_loss(self, batch):
        batch = move_to_device(batch, self.device)
        logits = self.model(input_ids=batch["input_ids"])["logits"]
        return local_loss(self.model, logits, batch["target_ids"], self.label_smoothing)


@StrategyFactory.register("sft")
class SFTStrategy(BaseStrategy):
    def __init__(self, model, device, label_smoothing: float = 0.0, **kwargs):
        super().__init__(model, device, **kwargs)
        self.label_smoothing = label_smoothing

    def compute_loss(self, batch):
        batch = move_to_device(batch, self.device)
        targets = batch["target_ids"].masked_fill(batch["loss_mask"] == 0, IGNORE_INDEX)
        logits = self.model(input_ids=batch["input_ids"])["logits"]
        return local_loss(self.model, logits, targets, self.label_smoothing)


@StrategyFactory.register("dpo")
class DPOStrategy(BaseStrategy):
    """``-logsigmoid(beta * ((pi_c - pi_r) - (ref_c - ref_r)))`` with chosen and rejected
    sequences run as one batch through the policy and through a frozen reference copy."""

    def __init__(self, model, device, beta: float = 0.1, reduction: str = "mean", **kwargs):
        super().__init__(model, device, **kwargs)
        self.ref_model = self._make_ref()
        self.beta, self.reduction = beta, reduction

    def compute_loss(self, batch):
        batch = move_to_device(batch, self.device)
        n = batch["chosen"].shape[0]
        ids = torch.cat([batch["chosen"], batch["rejected"]], dim=0)
        mask = torch.cat([batch["chosen_mask"], batch["rejected_mask"]], dim=0)
        pi = get_logprobs(self.model, ids, mask, self.reduction)
        with torch.no_grad():
            ref = get_logprobs(self.ref_model, ids, mask, self.reduction)
        margin = (pi[:n] - pi[n:]) - (ref[:n] - ref[n:])
        return -F.logsigmoid(self.beta * margin).mean()


@StrategyFactory.register("grpo")
class GRPOStrategy(BaseStrategy):
    """Clipped-ratio policy objective with group-normalised advantages and a squared
    log-ratio penalty; the frozen copy holds the old policy and is refreshed every
    ``sync_interval`` calls."""

    def __init__(self, model, device, clip_eps: float = 0.2, kl_coef: float = 0.01, group_size: int = 4,
                 reduction: str = "mean", sync_interval: int = 200, **kwargs):
        super().__init__(model, device, **kwargs)
        self.ref_model = self._make_ref()
        self.clip_eps, self.kl_coef, self.group_size = clip_eps, kl_coef, group_size
        self.reduction, self.sync_interval = reduction, sync_interval
        self._step = 0

    def sync_ref_model(self) -> None:
        state = self.executor.unwrap_model(self.model) if self.executor is not None else self.model.state_dict()
        if getattr(self.ref_model, "sharded_units", None) is not None:   # sharded block by block
            self.ref_model.sharded_units.load_full_state_dict(state)
        elif hasattr(self.ref_model, "scatter_named"):     # sliced / sharded copy: every rank takes its own pieces
            pieces = self.ref_model.scatter_named(state)
            with torch.no_grad():
                for p in self.ref_model.parameters():
                    p.copy_(pieces[id(p)])
        else:
            self.ref_model.load_state_dict(state)

    def _fold(self, batch):
        prompts, responses, masks, rewards = batch["prompts"], batch["responses"], batch["masks"], batch["rewards"]
        if responses.dim() == 2:
            B, G = responses.shape[0], self.group_size
            R = responses.shape[1] // G
            responses = responses[:, :G * R].reshape(B, G, R)
            masks = masks[:, :G * R].reshape(B, G, R)
            if rewards.dim() == 2 and rewards.shape[1] != G:
                rewards = rewards[:, :G * R].reshape(B, G, R).float().mean(dim=-1)
        return prompts, responses, masks, rewards.float()

    def compute_loss(self, batch):
        self._step += 1
        if self._step % self.sync_interval == 0:
            self.sync_ref_model()
        prompts, responses, masks, rewards = self._fold(move_to_device(batch, self.device))
        B, G, R = responses.shape
        prompt_rep = prompts.unsqueeze(1).expand(B, G, prompts.shape[-1]).reshape(B * G, -1)
        seqs = torch.cat([prompt_rep, responses.reshape(B * G, R)], dim=-1)
        full_mask = torch.cat([torch.ones_like(prompt_rep, dtype=masks.dtype), masks.reshape(B * G, R)], dim=-1)
        pi = get_logprobs(self.model, seqs, full_mask, self.reduction).view(B, G)
        with torch.no_grad():
            old = get_logprobs(self.ref_model, seqs, full_mask, self.reduction).view(B, G)
        adv = (rewards - rewards.mean(dim=-1, keepdim=True)) / (rewards.std(dim=-1, keepdim=True)
                                                              + torch.finfo(pi.dtype).eps)
        ratio = torch.exp(pi - old)
        clipped = torch.clamp(ratio, 1 - self.clip_eps, 1 + self.clip_eps)
        policy = -torch.min(ratio * adv, clipped * adv).mean()
        return policy + self.kl_coef * (pi - old).square().mean()
