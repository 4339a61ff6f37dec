"""FastAPI application: ``/health``, ``/stats``, ``/v1/chat/completions`` (OpenAI) and
``/v1/messages`` (Anthropic) on top of one ``InferenceEngine``
(reference: ``astrai/inference/api/server.py:30-169``).  ``/stats`` additionally reports
decode throughput and TTFT / latency percentiles."""

from __future__ import annotations

import logging
from contextlib import asynccontextmanager
from pathlib import Path
from typing import Any, Dict, List, Optional, Union

import torch
import uvicorn
from fastapi import FastAPI, HTTPException, Response
from pydantic import BaseModel, Field

from ...models import AutoModel
from ...tokenize import AutoTokenizer
from ..engine import InferenceEngine
from . import metrics
from .anthropic import AnthropicResponseBuilder
from .openai import OpenAIResponseBuilder
from .protocol import ProtocolHandler

log = logging.getLogger(__name__)
DEFAULT_PARAM_DIR = Path(__file__).resolve().parents[3] / "params"


class ChatMessage(BaseModel):
    role: str
    content: str


class ChatCompletionRequest(BaseModel):
    model: str = "astrai"
    messages: List[ChatMessage]
    temperature: Optional[float] = Field(default=1.0, ge=0.0, le=2.0)
    top_p: Optional[float] = Field(default=1.0, ge=0.0, le=1.0)
    top_k: Optional[int] = Field(default=50, ge=1)
    stream: Optional[bool] = False
    stop: Optional[Union[str, List[str]]] = None
    max_tokens: Optional[int] = Field(default=2048, ge=1)
    n: Optional[int] = Field(default=1, ge=1)
    presence_penalty: Optional[float] = Field(default=0.0, ge=-2.0, le=2.0)
    frequency_penalty: Optional[float] = Field(default=0.0, ge=-2.0, le=2.0)
    logit_bias: Optional[Dict[int, float]] = None
    user: Optional[str] = None


class AnthropicMessage(BaseModel):
    role: str
    content: Union[str, List[Dict[str, Any]]]


class MessagesRequest(BaseModel):
    model: str = "astrai"
    max_tokens: int = Field(default=1024, ge=1)
    messages: List[AnthropicMessage]
    system: Optional[str] = None
    temperature: Optional[float] = Field(default=1.0, ge=0.0, le=2.0)
    top_p: Optional[float] = Field(default=1.0, ge=0.0, le=1.0)
    top_k: Optional[int] = Field(default=50, ge=1)
    stream: Optional[bool] = False
    stop_sequences: Optional[List[str]] = None


def _load(param_path: Optional[Path], device: str, dtype: torch.dtype, int8: bool = False, tp: bool = False,
          adapter_path: Optional[Path] = None):
    root = Path(param_path) if param_path is not None else DEFAULT_PARAM_DIR
    if not root.exists():
        raise FileNotFoundError(f"Parameter directory not found: {root}")
    tokenizer = AutoTokenizer.from_pretrained(root)
    model = AutoModel.from_pretrained(root).to(device=device, dtype=dtype).eval()
    if adapter_path is not None:   # LoRA adapters are folded into the base weights before serving
        from ...models.components.lora import load_lora, merge_lora

        load_lora(model, str(adapter_path))
        merge_lora(model, unwrap=True)
    if tp:
        from ..tp import TPInferenceLM

        model = TPInferenceLM(model, int8=int8).eval()  # this rank's slices (quantised after slicing)
    elif int8:
        from ...ops.quant import quantize_model_int8

        quantize_model_int8(model)
    return model, tokenizer


def _create_engine(param_path: Optional[Path] = None, device: str = "cuda", dtype: torch.dtype = torch.bfloat16,
                   max_batch_size: int = 16, page_size: int = 16, max_seq_len: Optional[int] = None,
                   int8: bool = False, adapter_path: Optional[Path] = None) -> InferenceEngine:
    """Single-process engine, or rank 0 of a tensor-parallel group when a process group is up (the
    other ranks run ``serve_worker_rank``)."""
    import torch.distributed as dist

    tp = dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1
    model, tokenizer = _load(param_path, device, dtype, int8, tp, adapter_path)
    if not tp and next(model.parameters()).is_cuda and hasattr(model, "pack_parameters") and not int8:
        model.pack_parameters(with_grad=False)  # adjacent q/k/v and gate/up weights -> single GEMMs
    log.info("Model loaded on %s with dtype %s", device, dtype)
    return InferenceEngine(model=model, tokenizer=tokenizer, max_batch_size=max_batch_size, page_size=page_size,
                           max_seq_len=max_seq_len)


def serve_worker_rank(param_path: Optional[Path] = None, device: str = "cuda", dtype: torch.dtype = torch.bfloat16,
                      max_batch_size: int = 16, page_size: int = 16, max_seq_len: Optional[int] = None,
                      int8: bool = False, adapter_path: Optional[Path] = None) -> None:
    """Ranks > 0 of a tensor-parallel server: load the same weights, keep this rank's slice, replay
    the steps rank 0 announces until it shuts down."""
    from ..tp import serve_worker

    model, tokenizer = _load(param_path, device, dtype, int8, tp=True, adapter_path=adapter_path)
    serve_worker(model, tokenizer, max_batch_size=max_batch_size, max_seq_len=max_seq_len, page_size=page_size)


@asynccontextmanager
async def lifespan(app: FastAPI):
    config = getattr(app.state, "server_config", None) or {}
    if not config.get("_test", False):
        kwargs = {k: v for k, v in config.items() if not k.startswith("_")}
        app.state.engine = _create_engine(**kwargs)
    elif not hasattr(app.state, "engine"):
        app.state.engine = None
    yield
    if getattr(app.state, "engine", None):
        app.state.engine.shutdown()
        log.info("Inference engine shutdown complete")


app = FastAPI(title="khaosz_b200 inference server", version="0.1.0", lifespan=lifespan)
app.state.engine = None
app.state.server_config = {}


def _get_engine() -> InferenceEngine:
    engine = getattr(app.state, "engine", None)
    if engine is None:
        raise HTTPException(status_code=503, detail="Engine not initialized")
    return engine


@app.get("/health")
async def health():
    return {"status": "ok", "model_loaded": getattr(app.state, "engine", None) is not None}


@app.get("/stats")
async def get_stats():
    return _get_engine().get_stats()


@app.get("/metrics")
async def get_metrics():
    """Counters, gauges and the TTFT / inter-token / total latency histograms for a Prometheus scrape."""
    engine = _get_engine()
    return Response(content=metrics.render(engine.get_stats(), engine.get_histograms()), media_type=metrics.CONTENT_TYPE)


@app.post("/v1/chat/completions")
async def chat_completion(request: ChatCompletionRequest):
    return await ProtocolHandler(request, _get_engine(), OpenAIResponseBuilder()).handle()


@app.post("/v1/messages")
async def create_message(request: MessagesRequest):
    return await ProtocolHandler(request, _get_engine(), AnthropicResponseBuilder()).handle()


def run_server(host: str = "0.0.0.0", port: int = 8000, reload: bool = False, device: str = "cuda",
               dtype: torch.dtype = torch.bfloat16, param_path: Optional[Path] = None, max_batch_size: int = 16,
               page_size: int = 16, max_seq_len: Optional[int] = None, int8: bool = False,
               adapter_path: Optional[Path] = None) -> None:
    app.state.server_config = {"device": device, "dtype": dtype, "param_path": param_path,
                               "max_batch_size": max_batch_size, "page_size": page_size, "max_seq_len": max_seq_len,
                               "int8": int8, "adapter_path": adapter_path}
    uvicorn.run(app, host=host, port=port, reload=reload)
