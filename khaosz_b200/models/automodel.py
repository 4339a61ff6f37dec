"""``AutoModel``: registry of model classes keyed by ``model_type`` plus
``from_pretrained`` / ``save_pretrained`` (reference: ``astrai/model/automodel.py:43-91``)."""

from __future__ import annotations

import contextlib
from pathlib import Path
from typing import Union

import torch.nn as nn

from ..config.model_config import BaseModelConfig, ConfigFactory
from ..factory import BaseFactory
from ..serialization import CONFIG_FILE, WEIGHTS_FILE, load_model_config, load_model_weights, save_model

_INIT_FNS = ("normal_", "uniform_", "constant_", "ones_", "zeros_", "kaiming_uniform_", "kaiming_normal_",
             "xavier_uniform_", "xavier_normal_", "trunc_normal_")


@contextlib.contextmanager
def skip_random_init(active: bool = True):
    """Turn the ``torch.nn.init`` fillers into no-ops while a model that is about to be
    overwritten by a checkpoint is constructed."""
    if not active:
        yield
        return
    saved = {name: getattr(nn.init, name) for name in _INIT_FNS if hasattr(nn.init, name)}
    try:
        for name in saved:
            setattr(nn.init, name, lambda tensor, *a, **k: tensor)
        yield
    finally:
        for name, fn in saved.items():
            setattr(nn.init, name, fn)


class AutoModel(BaseFactory["AutoModel"], nn.Module):
    def __init__(self, config: BaseModelConfig):
        super().__init__()
        self.config = config

    @classmethod
    def from_pretrained(cls, path: Union[str, Path], disable_random_init: bool = True, strict: bool = True) -> nn.Module:
        root = Path(path)
        if not (root / CONFIG_FILE).exists():
            raise FileNotFoundError(f"Config file not found: {root / CONFIG_FILE}")
        config = ConfigFactory.load(load_model_config(str(root)))
        model_cls = AutoModel.get_component_class(config.model_type or ConfigFactory.DEFAULT_TYPE)
        with skip_random_init(disable_random_init):
            model = model_cls(config)
        if (root / WEIGHTS_FILE).exists():
            model.load_state_dict(load_model_weights(str(root)), strict=strict)
        return model

    def save_pretrained(self, save_directory: Union[str, Path]) -> None:
        save_model(config=self.config.to_dict(), state_dict=self.state_dict(), save_directory=str(save_directory))
