"""Schema of the JSONL -> token-shard preprocessing job.

The JSON layout (keys and defaults) is the user contract shared with the reference's
``astrai/config/preprocess_config.py:9-37``::

    {"version": 1,
     "input": {"sections": [{"field": "text", "action": "train"}]},
     "mask": {"user": "mask", "assistant": "train"}, "mask_default": "mask",
     "preprocessing": {"max_seq_len": 2048, "min_chars": 50, "max_chars": 2000000, "max_items": null},
     "output": {"domain_key": null, "storage_format": "bin", "max_tokens_per_shard": 100000000, "dtype": {}}}
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional

from .base import BaseConfig

STORAGE_FORMATS = ("bin", "h5")
MASK_ACTIONS = ("train", "mask")


@dataclass
class OutputConfig(BaseConfig):
    """Where and how shards are written. ``dtype`` overrides the int32 default per key."""

    domain_key: Optional[str] = None
    storage_format: str = "bin"
    max_tokens_per_shard: int = 100_000_000
    dtype: Dict[str, str] = field(default_factory=dict)

    def dtype_of(self, key: str, default: str = "int32") -> str:
        return (self.dtype or {}).get(key, default)


@dataclass
class ProcessingConfig(BaseConfig):
    """Length limits applied per item (characters for text mode, tokens after encoding)."""

    max_seq_len: int = 2048
    min_chars: int = 50
    max_chars: int = 2_000_000
    max_items: Optional[int] = None

    def keep_text(self, text: str) -> bool:
        return self.min_chars <= len(text) <= self.max_chars


@dataclass
class InputConfig(BaseConfig):
    """``sections``: ordered list of ``{field, action, template?, add_special_tokens?}``."""

    sections: Optional[List[Dict]] = None

    def iter_sections(self):
        return iter(self.sections or [])


@dataclass
class PipelineConfig(BaseConfig):
    version: int = 1
    input: InputConfig = field(default_factory=InputConfig)
    mask: Dict[str, str] = field(default_factory=dict)
    mask_default: str = "mask"
    preprocessing: ProcessingConfig = field(default_factory=ProcessingConfig)
    output: OutputConfig = field(default_factory=OutputConfig)

    def action_for_role(self, role: str) -> str:
        return (self.mask or {}).get(role, self.mask_default)
