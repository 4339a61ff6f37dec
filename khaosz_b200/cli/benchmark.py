"""Inference micro-benchmarks with CUDA-event timing.

``prefill`` / ``decode`` follow the recipe of the reference's ``scripts/tools/benchmark.py``
(random-init model, B x prompt tokens, 3 warm-ups, N timed trials); ``serve`` replays a
Poisson arrival trace of random-token prompts through ``InferenceEngine`` and reports decode
tokens/s and the median time to first token.
"""

from __future__ import annotations

import argparse
import json
import random
import threading
import time

import torch

from ..config import AutoRegressiveLMConfig
from ..inference import InferenceEngine
from ..inference.core.cache import KVCache
from ..models import AutoRegressiveLM

PRESETS = {
    "reference": dict(vocab_size=10000, dim=1536, n_heads=24, n_kv_heads=4, dim_ffn=6912, max_len=2048, n_layers=24,
                      norm_eps=1e-5),
    "1b": dict(vocab_size=32000, dim=2048, n_heads=16, n_kv_heads=4, dim_ffn=5632, max_len=4096, n_layers=24,
               norm_eps=1e-5, tie_weight=True),
}


class _IdTokenizer:
    """Token-id pass-through for synthetic load (prompts are lists of ids)."""

    stop_ids: list = []

    def encode(self, text, **_):
        return list(text) if not isinstance(text, str) else [ord(c) % 1000 for c in text]

    def decode(self, ids, **_):
        return " ".join(map(str, ids))


def build_model(preset: str, device: str, dtype):
    cfg = AutoRegressiveLMConfig(**PRESETS[preset])
    model = AutoRegressiveLM(cfg).to(device=device, dtype=dtype).eval()
    if device.startswith("cuda") and dtype == torch.bfloat16:
        model.pack_parameters(with_grad=False)
    return cfg, model


def _timed(fn, trials: int):
    total = 0.0
    for _ in range(trials):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        total += e0.elapsed_time(e1) / 1e3
    return total


@torch.inference_mode()
def bench_prefill(model, cfg, batch: int, prompt: int, trials: int, device):
    ids = lambda: torch.randint(0, cfg.vocab_size, (batch, prompt), device=device)
    for _ in range(3):
        model(ids())
    torch.cuda.synchronize()
    seconds = _timed(lambda: model(ids()), trials)
    return {"benchmark": "prefill", "batch": batch, "prompt": prompt, "tokens_per_s": batch * prompt * trials / seconds}


@torch.inference_mode()
def bench_decode(model, cfg, batch: int, prompt: int, gen: int, trials: int, page_size: int, device, dtype):
    n_pages = batch * ((prompt + gen + page_size - 1) // page_size + 1)
    cache = KVCache(cfg.n_layers, n_pages, page_size, cfg.n_kv_heads, cfg.dim // cfg.n_heads, device, dtype)
    names = [f"b{i}" for i in range(batch)]
    for n in names:
        cache.task_alloc(n, list(range(prompt + gen)))
    table = cache.make_table_tensor(names, device)

    def run():
        ids = torch.randint(0, cfg.vocab_size, (batch, prompt), device=device)
        model(ids, paged_cache=cache.bind(table, total_len=prompt), logits_rows=torch.arange(batch, device=device))
        tok = torch.randint(0, cfg.vocab_size, (batch, 1), device=device)
        for step in range(gen):
            pos = torch.full((batch, 1), prompt + step, device=device, dtype=torch.long)
            out = model(tok, paged_cache=cache.bind(table, seq_lens=pos.squeeze(1) + 1), position_ids=pos)
            tok = out["logits"][:, -1].argmax(-1, keepdim=True)

    run()
    torch.cuda.synchronize()
    seconds = _timed(run, trials)
    return {"benchmark": "decode", "batch": batch, "prompt": prompt, "generated": gen,
            "tokens_per_s": batch * gen * trials / seconds}


def bench_serve(model, cfg, requests: int, rate: float, min_prompt: int, max_prompt: int, gen: int, max_batch: int,
                page_size: int, seed: int, engine_cls=None, stop=None, budget_s: float = 0.0, warmup_requests: int = 4):
    """Replays a Poisson arrival trace through an engine with the reference's public interface
    (``engine.scheduler.add_task(prompt, max_tokens, temperature, top_p, top_k, stream_callback)``).
    ``engine_cls`` / ``stop`` select the engine under test: this package's by default, or the unmodified
    reference's ``InferenceEngine`` and its ``STOP`` sentinel.  Time to first token is taken here, from the
    stream callbacks, so that both engines are measured by the same clock.  ``budget_s`` > 0 ends the
    measurement after that many seconds whatever has finished (the row then says ``cut_at_budget``
    and the rates cover the tokens produced so far)."""
    from ..inference.core.task import STOP as OWN_STOP

    rng = random.Random(seed)
    engine_cls = engine_cls or InferenceEngine
    stop = OWN_STOP if stop is None else stop
    engine = engine_cls(model, _IdTokenizer(), max_batch_size=max_batch, max_seq_len=max_prompt + gen + 1,
                        max_prompt_len=max_prompt, page_size=page_size)
    done = threading.Semaphore(0)
    ttft, tokens_out = [], [0]

    def submit(length=None, tokens=None):
        n = rng.randint(min_prompt, max_prompt) if length is None else length
        prompt = [rng.randrange(cfg.vocab_size) for _ in range(n)]
        state = {"t0": time.time(), "first": None}

        def cb(tok):
            if tok is stop:
                done.release()
                return
            tokens_out[0] += 1
            if state["first"] is None:
                state["first"] = time.time() - state["t0"]
                ttft.append(state["first"])

        engine.scheduler.add_task(prompt, max_tokens=gen if tokens is None else tokens, temperature=1.0, top_p=1.0,
                                  top_k=1, stream_callback=cb)

    # a server is measured warm: a few short requests first (communicator set-up, first-use allocations,
    # the first recorded decode step), then the counters start again
    for i in range(max(0, warmup_requests)):
        submit(length=min_prompt + 16 * i, tokens=8)
    for _ in range(max(0, warmup_requests)):
        if not done.acquire(timeout=budget_s if budget_s > 0 else None):
            break
    ttft.clear()
    tokens_out[0] = 0
    t_start = time.time()

    for _ in range(requests):
        submit()
        if rate > 0:
            time.sleep(rng.expovariate(rate))
    cut = False
    for _ in range(requests):
        left = None if budget_s <= 0 else max(0.0, budget_s - (time.time() - t_start))
        if not done.acquire(timeout=left):
            cut = True
            break
    wall = time.time() - t_start
    stats = engine.get_stats()
    engine.shutdown()
    ttft.sort()
    pick = lambda q: ttft[min(len(ttft) - 1, int(q * len(ttft)))] if ttft else None
    return {"benchmark": "serve", "requests": requests, "arrival_rate_per_s": rate, "generated_per_request": gen,
            "output_tokens_per_s_wall": tokens_out[0] / wall, "decode_tokens_per_s_busy": stats.get("decode_tokens_per_s"),
            "ttft_p50_s": pick(0.50), "ttft_p99_s": pick(0.99), "wall_s": wall,
            "engine_ttft_p50_s": stats.get("ttft_p50_s"), "decode_graphs": stats.get("decode_graphs", 0),
            "cut_at_budget": cut, "tokens_generated": tokens_out[0], "first_tokens_seen": len(ttft)}


def reference_serve(a, dtype):
    """The same trace through the unmodified reference (``astrai.inference.InferenceEngine`` of the
    install under ``baseline/_ref``, its own model class, its own scheduler loop and kernels:
    ``astrai/inference/engine.py:93-288``, ``astrai/inference/core/scheduler.py:86-176``)."""
    import os
    import sys

    root = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "baseline", "_ref")
    if not os.path.isdir(os.path.join(root, "astrai")):
        return {"impl": "reference", "unavailable": "baseline/_ref/astrai is not installed"}
    try:
        import h5py  # noqa: F401
    except ImportError:
        import types

        sys.modules["h5py"] = types.ModuleType("h5py")   # imported by the reference at module import, never used here
    for name in [m for m in sys.modules if m == "astrai" or m.startswith("astrai.")]:
        del sys.modules[name]
    sys.path.insert(0, root)
    from astrai.config import AutoRegressiveLMConfig as RefConfig
    from astrai.inference import STOP as REF_STOP, InferenceEngine as RefEngine
    from astrai.model import AutoRegressiveLM as RefLM

    torch.manual_seed(a.seed)
    cfg = RefConfig(**PRESETS[a.preset])
    model = RefLM(cfg).to(device=a.device, dtype=dtype).eval()
    row = bench_serve(model, cfg, a.requests, a.rate, a.min_prompt, a.max_prompt, a.gen_length, a.max_batch_size,
                      a.page_size if a.page_size != 128 else 16, a.seed, engine_cls=RefEngine, stop=REF_STOP,
                      budget_s=a.budget_s, warmup_requests=a.warmup_requests)
    row["impl"] = "reference"
    return row


def parse_args(argv=None):
    p = argparse.ArgumentParser(description="prefill / decode / serving benchmarks")
    p.add_argument("mode", choices=["prefill", "decode", "serve", "all"], nargs="?", default="all")
    p.add_argument("--preset", choices=sorted(PRESETS), default="reference")
    p.add_argument("--batch_size", type=int, default=4)
    p.add_argument("--prompt_length", type=int, default=512)
    p.add_argument("--gen_length", type=int, default=128)
    p.add_argument("--trials", type=int, default=5)
    p.add_argument("--page_size", type=int, default=128)
    p.add_argument("--requests", type=int, default=256)
    p.add_argument("--rate", type=float, default=64.0, help="Poisson arrival rate (requests/s)")
    p.add_argument("--min_prompt", type=int, default=128)
    p.add_argument("--max_prompt", type=int, default=2048)
    p.add_argument("--max_batch_size", type=int, default=256)
    p.add_argument("--seed", type=int, default=3407)
    p.add_argument("--device", default="cuda")
    p.add_argument("--int8", action="store_true", help="int8 weight-only linears (per-channel scales)")
    p.add_argument("--warmup_requests", type=int, default=4,
                   help="serve mode: short requests served before the measured trace starts")
    p.add_argument("--budget_s", type=float, default=0.0,
                   help="serve mode: stop measuring after this many seconds and report what was produced so far")
    p.add_argument("--impl", choices=["khaosz_b200", "reference"], default="khaosz_b200",
                   help="serve mode: 'reference' drives the unmodified reference engine installed under baseline/_ref")
    return p.parse_args(argv)


def _tensor_parallel(a, dtype):
    """Under a multi-rank launcher (``torchrun``): rank 0 benchmarks, the others serve their slice."""
    import os

    import torch.distributed as dist

    from ..inference.tp import TPInferenceLM, serve_worker

    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    device = f"cuda:{local}"
    dist.init_process_group("nccl", device_id=torch.device(device))
    torch.manual_seed(a.seed)  # identical random weights on every rank
    cfg = AutoRegressiveLMConfig(**PRESETS[a.preset])
    model = AutoRegressiveLM(cfg).to(device=device, dtype=dtype).eval()
    model = TPInferenceLM(model, int8=a.int8).eval()
    page = a.page_size if a.page_size != 128 else 16
    if dist.get_rank() != 0:
        serve_worker(model, _IdTokenizer(), max_batch_size=a.max_batch_size, max_seq_len=a.max_prompt + a.gen_length + 1,
                     page_size=page)
    else:
        row = bench_serve(model, cfg, a.requests, a.rate, a.min_prompt, a.max_prompt, a.gen_length, a.max_batch_size,
                          page, a.seed, budget_s=a.budget_s, warmup_requests=a.warmup_requests)
        row.update(weights="int8" if a.int8 else "bf16", tensor_parallel=dist.get_world_size())
        print(json.dumps(row))
    dist.barrier()
    dist.destroy_process_group()


def main(argv=None):
    import os

    a = parse_args(argv)
    dtype = torch.bfloat16
    if int(os.environ.get("WORLD_SIZE", "1")) > 1:
        if a.mode != "serve":
            raise SystemExit("tensor-parallel benchmarking covers the serve mode")
        return _tensor_parallel(a, dtype)
    if a.impl == "reference":
        if a.mode != "serve":
            raise SystemExit("the reference arm covers the serve mode (its own scripts/tools/benchmark.py has the others)")
        row = reference_serve(a, dtype)
        row["weights"] = "bf16"
        print(json.dumps(row))
        return [row]
    cfg, model = build_model(a.preset, a.device, dtype)
    if a.int8:
        from ..ops.quant import quantize_model_int8

        quantize_model_int8(model)
    out = []
    if a.mode in ("prefill", "all"):
        out.append(bench_prefill(model, cfg, a.batch_size, a.prompt_length, a.trials, a.device))
    if a.mode in ("decode", "all"):
        out.append(bench_decode(model, cfg, a.batch_size, a.prompt_length, a.gen_length, a.trials, a.page_size,
                                a.device, dtype))
    if a.mode == "serve":
        out.append(bench_serve(model, cfg, a.requests, a.rate, a.min_prompt, a.max_prompt, a.gen_length,
                               a.max_batch_size, a.page_size if a.page_size != 128 else 16, a.seed, budget_s=a.budget_s,
                               warmup_requests=a.warmup_requests))
    for row in out:
        row["weights"] = "int8" if a.int8 else "bf16"
        print(json.dumps(row))
    return out


if __name__ == "__main__":
    main()
