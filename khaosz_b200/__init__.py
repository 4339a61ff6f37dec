"""khaosz_b200: a Blackwell-native (sm_100a) transformer training and inference framework
with the capabilities of ViperEkura/KHAOSZ (``astrai``)."""

__version__ = "0.1.0"

from .config import AutoRegressiveLMConfig, EncoderConfig, TrainConfig
from .data import DatasetFactory
from .factory import BaseFactory
from .inference import GenerationRequest, InferenceEngine
from .models import AutoModel, AutoRegressiveLM
from .tokenize import AutoTokenizer
from .trainer import CallbackFactory, SchedulerFactory, StrategyFactory, Trainer

__all__ = ["AutoRegressiveLM", "AutoRegressiveLMConfig", "EncoderConfig", "TrainConfig", "DatasetFactory",
           "AutoTokenizer", "GenerationRequest", "InferenceEngine", "Trainer", "CallbackFactory", "StrategyFactory",
           "SchedulerFactory", "BaseFactory", "AutoModel"]
