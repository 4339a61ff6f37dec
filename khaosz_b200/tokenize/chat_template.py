"""Jinja2 chat templates (reference: ``astrai/tokenize/chat_template.py:8-74``)."""

from __future__ import annotations

from typing import Any, Dict, List, Optional

from jinja2 import Template

Message = Dict[str, str]


class ChatTemplate:
    """A compiled Jinja2 template rendered with ``messages`` (+ optional ``system_prompt``);
    variable precedence: call-time variables > ``special_tokens`` > ``default_variables``."""

    def __init__(self, name: str = "", template_str: str = "", description: str = "",
                 default_variables: Optional[Dict[str, Any]] = None, special_tokens: Optional[Dict[str, str]] = None):
        self.name, self.template_str, self.description = name, template_str, description
        self.default_variables = dict(default_variables or {})
        self.special_tokens = dict(special_tokens or {})
        self._compiled = Template(template_str)

    @classmethod
    def from_string(cls, template_str: str, description: str = "", default_variables: Optional[Dict[str, Any]] = None,
                    special_tokens: Optional[Dict[str, str]] = None) -> "ChatTemplate":
        return cls("", template_str, description, default_variables, special_tokens)

    def render(self, messages: List[Message], system_prompt: Optional[str] = None, **extra_variables: Any) -> str:
        scope = {**self.default_variables, **self.special_tokens, **extra_variables, "messages": messages}
        if system_prompt is not None:
            scope["system_prompt"] = system_prompt
        return self._compiled.render(**scope)
