"""JSONL record -> ``{sequence, domain, loss_mask?}``.

One config-driven builder covers chat, instruction and plain-text data.  Each entry of
``input.sections`` names a JSONL field and how its tokens enter the loss:

    {"field": "messages", "action": "$role", "template": true}      # chat: per-message template,
                                                                     # role looked up in config.mask
    {"field": "prompt", "action": "mask", "add_special_tokens": true}
    {"field": "text", "action": "train"}

Behaviour follows ``astrai/preprocessing/builder.py:86-159``: a masked BOS is prepended for
template configs, plain-text-only configs apply the character limits, sequences are cut to
``max_seq_len`` and ``loss_mask`` is dropped when every token trains.
"""

from __future__ import annotations

from abc import ABC, abstractmethod
from typing import List, Optional, Tuple

from ..factory import BaseFactory

DEFAULT_DOMAIN = "__default__"


class BaseMaskBuilder(ABC):
    @abstractmethod
    def build(self, item: dict, config, tokenizer) -> Optional[dict]:
        """Return ``{sequence, domain, loss_mask?}`` or ``None`` to skip the record."""


class MaskBuilderFactory(BaseFactory[BaseMaskBuilder]):
    @classmethod
    def _validate_component(cls, component_cls: type) -> None:
        if not (isinstance(component_cls, type) and issubclass(component_cls, BaseMaskBuilder)):
            raise TypeError(f"{getattr(component_cls, '__name__', component_cls)} must inherit from BaseMaskBuilder")


def domain_of(item: dict, domain_key: Optional[str]) -> str:
    value = item.get(domain_key, DEFAULT_DOMAIN) if domain_key else DEFAULT_DOMAIN
    return value if isinstance(value, str) else DEFAULT_DOMAIN


def resolve_action(action: str, role: str, config) -> str:
    if action == "$role":
        return (config.mask or {}).get(role, config.mask_default)
    return action


@MaskBuilderFactory.register("sectioned")
class SectionedMaskBuilder(BaseMaskBuilder):
    def _chat_section(self, messages, action: str, config, tokenizer) -> List[Tuple[List[int], int]]:
        pieces = []
        for msg in messages:
            if not isinstance(msg, dict):        # a malformed turn is dropped, the rest of the dialogue kept
                continue
            text = tokenizer.apply_chat_template([msg], tokenize=False, add_generation_prompt=False)
            ids = tokenizer.encode(text, add_special_tokens=False)
            pieces.append((ids, int(resolve_action(action, msg.get("role", ""), config) == "train")))
        return pieces

    def build(self, item: dict, config, tokenizer) -> Optional[dict]:
        sections = config.input.sections
        if not sections:
            return None
        templated = any(sec.get("template") for sec in sections)
        text_only = not templated and all(sec["action"] == "train" for sec in sections)
        limits = config.preprocessing

        ids: List[int] = []
        mask: List[int] = []
        if templated and tokenizer.bos_token_id is not None:
            ids.append(tokenizer.bos_token_id)
            mask.append(0)
        for n, sec in enumerate(sections):
            use_template = bool(sec.get("template", False))
            if use_template:
                messages = item.get(sec["field"])
                if not isinstance(messages, list) or not messages:
                    continue
                pieces = self._chat_section(messages, sec["action"], config, tokenizer)
            else:
                text = str(item.get(sec["field"], ""))
                if not text.strip():
                    continue
                if text_only and ((limits.min_chars > 0 and len(text) < limits.min_chars) or len(text) > limits.max_chars):
                    continue
                add_special = sec.get("add_special_tokens", n == 0)
                pieces = [(tokenizer.encode(text, add_special_tokens=add_special), int(sec["action"] == "train"))]
            for piece_ids, flag in pieces:
                ids.extend(piece_ids)
                mask.extend([flag] * len(piece_ids))

        ids = ids[: limits.max_seq_len]
        mask = mask[: len(ids)]
        if not ids or (templated and len(ids) <= 1):
            return None
        out = {"sequence": ids, "domain": domain_of(item, config.output.domain_key)}
        if not all(mask):
            out["loss_mask"] = mask
        return out
