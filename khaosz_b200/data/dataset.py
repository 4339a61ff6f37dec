"""Sliding-window datasets over a token ``Store`` (reference: ``astrai/dataset/dataset.py``).

Window ``i`` covers ``[begin, end)`` with ``begin = min(i * stride, total - 1 - window)`` and
``end = min(begin + window, total - 1)``; ``len = (total - 1 - window) // stride + 1`` (0 when
the data is not longer than one window).  Each dataset type is a small table of
``output name -> (storage key, shift, dtype)``.
"""

from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import torch
from torch import Tensor
from torch.utils.data import Dataset

from ..factory import BaseFactory
from .storage import Store, StoreFactory, detect_format

Field = Tuple[str, int, Optional[torch.dtype]]  # storage key, shift, cast (None = as stored)


class BaseDataset(Dataset):
    FIELDS: Dict[str, Field] = {}

    def __init__(self, window_size: int, stride: int):
        super().__init__()
        self.window_size, self.stride = window_size, stride
        self.storage: Optional[Store] = None
        self._load_path: Optional[str] = None

    @property
    def required_keys(self) -> List[str]:
        return list(dict.fromkeys(key for key, _, _ in self.FIELDS.values()))

    def load(self, load_path: str, storage_type: Optional[str] = None) -> None:
        kind = storage_type or detect_format(load_path)
        self.storage = StoreFactory.create(kind)
        self._load_path = load_path
        self.storage.load(load_path)
        missing = [k for k in self.required_keys if k not in set(self.storage.keys)]
        if missing:
            raise KeyError(f"{type(self).__name__} requires keys {self.required_keys}; storage at {load_path} has "
                           f"{sorted(self.storage.keys)} (missing {missing})")

    @property
    def count(self) -> int:
        return len(self.storage) if self.storage is not None else 0

    @property
    def keys(self) -> List[str]:
        return self.storage.keys if self.storage is not None else []

    def get_index(self, index: int) -> Tuple[int, int]:
        if self.storage is None:
            raise RuntimeError("Dataset not loaded, call load() first")
        total = len(self.storage)
        if total <= self.window_size:
            raise ValueError(f"Data too short: {total} tokens <= window_size {self.window_size}")
        begin = min(index * self.stride, total - 1 - self.window_size)
        return begin, min(begin + self.window_size, total - 1)

    def __len__(self) -> int:
        total = self.count
        return 0 if total <= self.window_size else (total - 1 - self.window_size) // self.stride + 1

    def __getitem__(self, index: int) -> Dict[str, Tensor]:
        begin, end = self.get_index(index)
        sample = {}
        for name, (key, shift, dtype) in self.FIELDS.items():
            t = self.storage.fetch(begin + shift, end + shift, key)
            sample[name] = t if dtype is None else t.to(dtype)
        return sample


class DatasetFactory(BaseFactory[BaseDataset]):
    @classmethod
    def _validate_component(cls, dataset_cls: type) -> None:
        if not (isinstance(dataset_cls, type) and issubclass(dataset_cls, BaseDataset)):
            raise TypeError(f"{getattr(dataset_cls, '__name__', dataset_cls)} must inherit from BaseDataset")

    @classmethod
    def create(cls, train_type: str, window_size: int, stride: int) -> BaseDataset:
        return super().create(train_type, window_size, stride)

    @classmethod
    def load(cls, train_type: str, load_path: str, window_size: int, stride: Optional[int] = None,
             storage_type: Optional[str] = None) -> BaseDataset:
        ds = cls.create(train_type, window_size, window_size if stride is None else stride)
        ds.load(load_path, storage_type=storage_type)
        return ds

    @classmethod
    def available_types(cls) -> list:
        return cls.list_registered()


@DatasetFactory.register("seq")
class SEQDataset(BaseDataset):
    """Next-token pre-training: targets are the inputs shifted by one."""

    FIELDS = {"input_ids": ("sequence", 0, torch.long), "target_ids": ("sequence", 1, torch.long)}


@DatasetFactory.register("sft")
class SFTDataset(BaseDataset):
    FIELDS = {"input_ids": ("sequence", 0, torch.long), "target_ids": ("sequence", 1, torch.long),
              "loss_mask": ("loss_mask", 1, torch.bool)}


@DatasetFactory.register("dpo")
class DPODataset(BaseDataset):
    FIELDS = {"chosen": ("chosen", 0, torch.long), "rejected": ("rejected", 0, torch.long),
              "chosen_mask": ("chosen_mask", 0, torch.bool), "rejected_mask": ("rejected_mask", 0, torch.bool)}


@DatasetFactory.register("grpo")
class GRPODataset(BaseDataset):
    FIELDS = {"prompts": ("prompts", 0, torch.long), "responses": ("responses", 0, torch.long),
              "masks": ("masks", 0, torch.bool), "rewards": ("rewards", 0, None)}
