"""Dataclass configs that round-trip through plain dicts / JSON.

Same contract as the reference's ``astrai/config/base.py:8-98``: only JSON-safe fields are
emitted, unknown keys are ignored on load, missing keys take the dataclass default, and
scalars are coerced to the annotated type (``3.0 -> 3`` for an ``int`` field, nested dicts
to nested configs).
"""

from __future__ import annotations

import dataclasses
import json
import typing
from pathlib import Path
from typing import Any, Dict, Union


def _jsonable(value: Any):
    """Return (True, json-safe value) or (False, None) when the value cannot be stored."""
    if value is None or isinstance(value, (str, bool, int, float)):
        return True, value
    if isinstance(value, BaseConfig):
        return True, value.to_dict()
    if dataclasses.is_dataclass(value) and not isinstance(value, type):
        out = {}
        for f in dataclasses.fields(value):
            item = getattr(value, f.name)
            out[f.name] = list(item) if isinstance(item, tuple) else item
        return True, out
    if isinstance(value, (list, tuple, dict)):
        candidate = list(value) if isinstance(value, tuple) else value
        try:
            json.dumps(candidate)
        except (TypeError, ValueError):
            return False, None
        return True, candidate
    return False, None


def _strip_optional(tp):
    args = typing.get_args(tp)
    if typing.get_origin(tp) is not None and args:
        concrete = [a for a in args if a is not type(None)]
        return concrete[0] if concrete else None
    return tp


def _convert(value: Any, tp) -> Any:
    if tp is None or not isinstance(tp, type):
        return value
    number = isinstance(value, (int, float)) and not isinstance(value, bool)
    if tp is int and number:
        return int(value)
    if tp is float and number:
        return float(value)
    if isinstance(value, dict) and issubclass(tp, BaseConfig):
        return tp.from_dict(value)
    return value


@dataclasses.dataclass
class BaseConfig:
    def to_dict(self) -> Dict[str, Any]:
        out: Dict[str, Any] = {}
        for f in dataclasses.fields(self):
            ok, val = _jsonable(getattr(self, f.name))
            if ok:
                out[f.name] = val
        return out

    @classmethod
    def from_dict(cls, data: Dict[str, Any]):
        hints = typing.get_type_hints(cls)
        obj = cls.__new__(cls)  # bypass __init__/__post_init__: partial dicts are legal
        for f in dataclasses.fields(cls):
            if f.name in data:
                value = _convert(data[f.name], _strip_optional(hints.get(f.name)))
            elif f.default is not dataclasses.MISSING:
                value = f.default
            elif f.default_factory is not dataclasses.MISSING:
                value = f.default_factory()
            else:
                value = None
            object.__setattr__(obj, f.name, value)
        return obj

    @classmethod
    def from_json(cls, path: Union[str, Path]):
        return cls.from_dict(json.loads(Path(path).read_text(encoding="utf-8")))

    def to_json(self, path: Union[str, Path]) -> None:
        Path(path).write_text(json.dumps(self.to_dict(), indent=2, ensure_ascii=False), encoding="utf-8")
