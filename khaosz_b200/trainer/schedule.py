"""Learning-rate schedules: warm-up + cosine decay, and warm-up + SGDR restarts.

Factor curves match ``astrai/trainer/schedule.py:75-194`` (first LR is ``min_rate * base``;
the extra hyper-parameters travel in ``state_dict``).  Each schedule is a pure function of
the step, wrapped in a ``torch`` ``LRScheduler``.
"""

from __future__ import annotations

import math
from typing import Dict, List

from torch.optim.lr_scheduler import LRScheduler

from ..factory import BaseFactory


class BaseScheduler(LRScheduler):
    """``factor(step)`` scales every base LR; ``HYPER`` lists attributes kept in checkpoints."""

    HYPER: tuple = ()

    def factor(self, step: int) -> float:
        raise NotImplementedError

    def get_lr(self) -> List[float]:
        f = self.factor(self.last_epoch)
        return [base * f for base in self.base_lrs]

    def state_dict(self) -> Dict:
        state = super().state_dict()
        state.update({name: getattr(self, name) for name in self.HYPER})
        return state

    def load_state_dict(self, state_dict: Dict) -> None:
        state_dict = dict(state_dict)
        for name in self.HYPER:
            if name in state_dict:
                setattr(self, name, state_dict.pop(name))
        super().load_state_dict(state_dict)


class SchedulerFactory(BaseFactory[BaseScheduler]):
    @classmethod
    def _validate_component(cls, scheduler_cls: type) -> None:
        if not (isinstance(scheduler_cls, type) and issubclass(scheduler_cls, BaseScheduler)):
            raise TypeError(f"{getattr(scheduler_cls, '__name__', scheduler_cls)} must inherit from BaseScheduler")

    @classmethod
    def create(cls, optimizer, schedule_type: str = "none", **kwargs) -> BaseScheduler:
        return super().create(schedule_type, optimizer, **kwargs)

    @classmethod
    def available_types(cls) -> list:
        return cls.list_registered()


def _warmup(step: int, warmup_steps: int, min_rate: float) -> float:
    return max(min_rate, step / warmup_steps)


@SchedulerFactory.register("cosine")
class CosineScheduler(BaseScheduler):
    HYPER = ("warmup_steps", "lr_decay_steps", "min_rate", "total_steps")

    def __init__(self, optimizer, warmup_steps: int, lr_decay_steps: int, min_rate: float = 0.05,
                 last_epoch: int = -1):
        self.warmup_steps, self.lr_decay_steps, self.min_rate = warmup_steps, lr_decay_steps, min_rate
        self.total_steps = warmup_steps + lr_decay_steps
        super().__init__(optimizer, last_epoch)

    def factor(self, step: int) -> float:
        if step < self.warmup_steps:
            return _warmup(step, self.warmup_steps, self.min_rate)
        progress = min((step - self.warmup_steps) / max(self.lr_decay_steps, 1), 1.0)
        return max(self.min_rate, 0.5 * (1.0 + math.cos(math.pi * progress)))


@SchedulerFactory.register("sgdr")
class SGDRScheduler(BaseScheduler):
    HYPER = ("warmup_steps", "cycle_length", "min_rate", "t_mult")

    def __init__(self, optimizer, warmup_steps: int, cycle_length: int, min_rate: float = 0.05, t_mult: int = 2,
                 last_epoch: int = -1):
        self.warmup_steps, self.cycle_length, self.min_rate, self.t_mult = warmup_steps, cycle_length, min_rate, t_mult
        super().__init__(optimizer, last_epoch)

    def factor(self, step: int) -> float:
        if step < self.warmup_steps:
            return _warmup(step, self.warmup_steps, self.min_rate)
        pos, length = step - self.warmup_steps, self.cycle_length
        while pos >= length:  # walk the geometrically growing cycles
            pos -= length
            length *= self.t_mult
        return self.min_rate + (1 - self.min_rate) * 0.5 * (1 + math.cos(math.pi * pos / length))
