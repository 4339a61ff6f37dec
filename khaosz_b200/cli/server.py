"""Inference server CLI (reference: ``scripts/tools/server.py:9-68``) with ``--page_size``."""

from __future__ import annotations

import argparse
from pathlib import Path

import torch

DTYPES = {"bfloat16": torch.bfloat16, "float16": torch.float16, "float32": torch.float32}


def parse_args(argv=None):
    p = argparse.ArgumentParser(description="OpenAI / Anthropic compatible inference server")
    p.add_argument("--host", default="0.0.0.0")
    p.add_argument("--port", type=int, default=8000)
    p.add_argument("--reload", action="store_true")
    p.add_argument("--param_path", type=Path, default=None, help="Directory with config, weights and tokenizer")
    p.add_argument("--device", default="cuda")
    p.add_argument("--dtype", default="bfloat16", choices=sorted(DTYPES))
    p.add_argument("--max_batch_size", type=int, default=16)
    p.add_argument("--page_size", type=int, default=16, help="KV-cache page size in tokens")
    p.add_argument("--max_seq_len", type=int, default=None)
    return p.parse_args(argv)


def main(argv=None):
    from ..inference.api import run_server

    a = parse_args(argv)
    run_server(host=a.host, port=a.port, reload=a.reload, device=a.device, dtype=DTYPES[a.dtype],
               param_path=a.param_path, max_batch_size=a.max_batch_size, page_size=a.page_size,
               max_seq_len=a.max_seq_len)


if __name__ == "__main__":
    main()
