from .base import BaseConfig
from .model_config import AutoRegressiveLMConfig, BaseModelConfig, ConfigFactory, EncoderConfig
from .pipeline_config import InputConfig, OutputConfig, PipelineConfig, ProcessingConfig
from .train_config import TrainConfig

__all__ = ["BaseConfig", "BaseModelConfig", "AutoRegressiveLMConfig", "EncoderConfig", "ConfigFactory",
           "TrainConfig", "InputConfig", "OutputConfig", "PipelineConfig", "ProcessingConfig"]
