"""khaosz_b200: a Blackwell-native (sm_100a) transformer training and inference framework
with the capabilities of ViperEkura/KHAOSZ (``astrai``)."""

__version__ = "0.1.0"

from .config import AutoRegressiveLMConfig, EncoderConfig, TrainConfig
from .factory import BaseFactory
from .models import AutoModel, AutoRegressiveLM

__all__ = ["AutoRegressiveLM", "AutoRegressiveLMConfig", "EncoderConfig", "TrainConfig", "BaseFactory", "AutoModel"]
