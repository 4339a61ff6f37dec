"""Inference server CLI (reference: ``scripts/tools/server.py:9-68``) with ``--page_size``,
``--int8`` (weight-only int8 linears) and ``--tp_size N`` (one process per GPU: rank 0 serves HTTP
and schedules, the other ranks replay its steps on their slice of the model)."""

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
    p.add_argument("--int8", action="store_true", help="int8 weight-only linears (per-channel scales)")
    p.add_argument("--adapter_path", type=Path, default=None,
                   help="LoRA adapter directory (adapter_model.safetensors + adapter_config.json), merged at load")
    p.add_argument("--tp_size", type=int, default=1, help="tensor-parallel ranks (GPUs) of one server")
    p.add_argument("--master_addr", default="127.0.0.1")
    p.add_argument("--master_port", default="29560")
    return p.parse_args(argv)


def _rank_main(a) -> None:
    """One rank of a tensor-parallel server (runs inside ``setup_parallel``)."""
    import torch.distributed as dist

    from ..inference.api import run_server
    from ..inference.api.server import serve_worker_rank
    from ..parallel.setup import get_current_device

    device = get_current_device() if a.device == "cuda" else a.device
    common = dict(device=device, dtype=DTYPES[a.dtype], param_path=a.param_path, max_batch_size=a.max_batch_size,
                  page_size=a.page_size, max_seq_len=a.max_seq_len, int8=a.int8, adapter_path=a.adapter_path)
    if dist.get_rank() == 0:
        run_server(host=a.host, port=a.port, reload=False, **common)
    else:
        serve_worker_rank(**common)


def main(argv=None):
    from ..inference.api import run_server

    a = parse_args(argv)
    if a.tp_size > 1:
        from ..parallel import spawn_parallel_fn

        spawn_parallel_fn(_rank_main, world_size=a.tp_size, backend="nccl" if a.device == "cuda" else "gloo",
                          master_addr=a.master_addr, master_port=a.master_port,
                          device_type="cuda" if a.device == "cuda" else "cpu", a=a)
        return
    run_server(host=a.host, port=a.port, reload=a.reload, device=a.device, dtype=DTYPES[a.dtype],
               param_path=a.param_path, max_batch_size=a.max_batch_size, page_size=a.page_size,
               max_seq_len=a.max_seq_len, int8=a.int8, adapter_path=a.adapter_path)


if __name__ == "__main__":
    main()
