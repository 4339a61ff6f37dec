"""``AutoTokenizer``: a HuggingFace ``tokenizers`` model plus special-token map and chat
template, stored as ``tokenizer.json`` + ``tokenizer_config.json {special_tokens, chat_template}``
(reference: ``astrai/tokenize/tokenizer.py:14-264``).

Dynamic attributes: ``tok.<name>`` -> the special token string, ``tok.<name>_id`` -> its id,
``tok.stop_ids`` -> ids of every special token.
"""

from __future__ import annotations

import json
from pathlib import Path
from typing import Dict, List, Optional, Union

from tokenizers import Tokenizer

from .chat_template import ChatTemplate

TOKENIZER_FILE = "tokenizer.json"
TOKENIZER_CONFIG = "tokenizer_config.json"


class AutoTokenizer:
    TOKENIZER_CLASSES: Dict[str, type] = {}

    def __init__(self, path: Optional[Union[str, Path]] = None, special_token_map: Optional[Dict[str, str]] = None,
                 chat_template: Optional[str] = None):
        self._tokenizer: Optional[Tokenizer] = None
        self._chat_template: Optional[ChatTemplate] = None
        self._special_token_map: Dict[str, str] = dict(special_token_map or {})
        if chat_template:
            self.set_chat_template(chat_template)
        if path:
            self.load(path)

    # -- persistence ------------------------------------------------------------------------
    def load(self, path: Union[str, Path]) -> None:
        root = Path(path)
        self._tokenizer = Tokenizer.from_file(str(root / TOKENIZER_FILE))
        cfg_path = root / TOKENIZER_CONFIG
        if cfg_path.exists():
            cfg = json.loads(cfg_path.read_text(encoding="utf-8"))
            self._special_token_map.update(cfg.get("special_tokens", {}))
            if cfg.get("chat_template"):
                self.set_chat_template(cfg["chat_template"])

    @classmethod
    def from_pretrained(cls, path: Union[str, Path]) -> "AutoTokenizer":
        root = Path(path)
        if not (root / TOKENIZER_FILE).exists():
            raise FileNotFoundError(f"Tokenizer file not found: {root / TOKENIZER_FILE}")
        tok = cls(root)
        if tok._tokenizer is None:
            raise RuntimeError(f"Failed to load tokenizer from {root}")
        return tok

    def save_pretrained(self, save_path: str) -> None:
        self._require()
        root = Path(save_path)
        root.mkdir(parents=True, exist_ok=True)
        self._tokenizer.save(str(root / TOKENIZER_FILE))
        cfg = {"special_tokens": self._special_token_map}
        if self._chat_template is not None:
            cfg["chat_template"] = self._chat_template.template_str
        (root / TOKENIZER_CONFIG).write_text(json.dumps(cfg, ensure_ascii=False, indent=2), encoding="utf-8")

    @classmethod
    def register_tokenizer(cls, name: str, tokenizer_class: type) -> None:
        cls.TOKENIZER_CLASSES[name] = tokenizer_class

    # -- encode / decode --------------------------------------------------------------------
    def _require(self) -> Tokenizer:
        if self._tokenizer is None:
            raise RuntimeError("Tokenizer not initialized. Load or create a tokenizer first.")
        return self._tokenizer

    def encode(self, tokens: Union[str, List[str]], out_ids: bool = True, is_pretokenized: bool = False,
               add_special_tokens: bool = True) -> List:
        tk = self._require()
        pick = (lambda e: e.ids) if out_ids else (lambda e: e.tokens)
        if isinstance(tokens, str):
            return pick(tk.encode(tokens, is_pretokenized=is_pretokenized, add_special_tokens=add_special_tokens))
        batch = tk.encode_batch(tokens, is_pretokenized=is_pretokenized, add_special_tokens=add_special_tokens)
        return [pick(e) for e in batch]

    def decode(self, tokens: List[int], skip_special_tokens: bool = True) -> str:
        return self._require().decode(tokens, skip_special_tokens=skip_special_tokens)

    def __len__(self) -> int:
        return self._tokenizer.get_vocab_size() if self._tokenizer is not None else 0

    @property
    def vocab_size(self) -> int:
        return len(self)

    # -- special tokens ---------------------------------------------------------------------
    def __getattr__(self, key: str):
        if key.startswith("_"):
            raise AttributeError(key)
        tokens = self.__dict__.get("_special_token_map", {})
        tk = self.__dict__.get("_tokenizer")
        if key == "stop_ids":
            if tk is None:
                return []
            ids = (tk.token_to_id(text) for text in tokens.values())
            return [i for i in ids if i is not None]
        if key.endswith("_id"):
            text = tokens.get(key[:-3])
            if text is None:
                return None
            if tk is None:
                raise RuntimeError("Tokenizer not loaded, cannot convert token to id.")
            return tk.token_to_id(text)
        if key in tokens:
            return tokens[key]
        raise AttributeError(f"'{type(self).__name__}' object has no attribute '{key}'")

    # -- chat -------------------------------------------------------------------------------
    def set_chat_template(self, template: Union[str, ChatTemplate]) -> None:
        if isinstance(template, ChatTemplate):
            self._chat_template = template
        elif isinstance(template, str):
            self._chat_template = ChatTemplate.from_string(template)
        else:
            raise ValueError("Invalid template type, must be str or ChatTemplate.")

    def apply_chat_template(self, messages: List[Dict[str, str]], system_prompt: Optional[str] = None,
                            tokenize: bool = True, add_generation_prompt: bool = True, **kwargs):
        if self._chat_template is None:
            raise RuntimeError("Chat template not set. Use set_chat_template() to set a template first.")
        if system_prompt:
            messages = [{"role": "system", "content": system_prompt}, *messages]
        text = self._chat_template.render(messages=messages, add_generation_prompt=add_generation_prompt, **kwargs)
        return self.encode(text) if tokenize else text
