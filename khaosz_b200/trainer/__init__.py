from .callbacks import (CallbackFactory, CheckpointCallback, DeviceHealthCallback, GradientCheckpointingCallback,
                        GradientClippingCallback, MetricLoggerCallback, ProgressBarCallback, ThroughputCallback,
                        TrainCallback, ValidationCallback)
from .context import TrainContext, TrainContextBuilder
from .optim import FusedAdamW, Muon
from .schedule import BaseScheduler, CosineScheduler, SchedulerFactory, SGDRScheduler
from .strategy import (BaseStrategy, DPOStrategy, GRPOStrategy, SEQStrategy, SFTStrategy, StrategyFactory,
                       create_ref_model, get_logprobs)
from .trainer import Trainer

__all__ = ["CallbackFactory", "CheckpointCallback", "DeviceHealthCallback", "ThroughputCallback", "GradientCheckpointingCallback", "GradientClippingCallback",
           "MetricLoggerCallback", "ProgressBarCallback", "TrainCallback", "ValidationCallback", "TrainContext",
           "TrainContextBuilder", "FusedAdamW", "Muon", "BaseScheduler", "CosineScheduler", "SchedulerFactory",
           "SGDRScheduler", "BaseStrategy", "DPOStrategy", "GRPOStrategy", "SEQStrategy", "SFTStrategy",
           "StrategyFactory", "create_ref_model", "get_logprobs", "Trainer"]
