from .chat_template import ChatTemplate
from .tokenizer import AutoTokenizer

__all__ = ["AutoTokenizer", "ChatTemplate"]
