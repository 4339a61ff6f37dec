from .anthropic import AnthropicResponseBuilder
from .openai import OpenAIResponseBuilder
from .protocol import GenContext, ProtocolHandler, ResponseBuilder, StopChecker, StopInfo, sse_done, sse_event
from .server import (AnthropicMessage, ChatCompletionRequest, ChatMessage, MessagesRequest, app, run_server)

__all__ = ["AnthropicResponseBuilder", "OpenAIResponseBuilder", "GenContext", "ProtocolHandler", "ResponseBuilder",
           "StopChecker", "StopInfo", "sse_done", "sse_event", "AnthropicMessage", "ChatCompletionRequest",
           "ChatMessage", "MessagesRequest", "app", "run_server"]
