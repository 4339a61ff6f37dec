#!/usr/bin/env python
"""Headline benchmark: pre-training throughput (tokens/s) of the 1B-class decoder.

Model: 24 layers, d_model 2048, 16 query / 4 KV heads (head_dim 128), SwiGLU ffn 5632, vocab
32000, tied embeddings, bf16.  Step = one optimizer step = 8 micro-batches of 4 x 2048
tokens per GPU (weak scaling: per-GPU work is fixed), AdamW(lr 3e-4, betas (0.9, 0.95),
wd 0.01), label smoothing 0.05, gradient clip 1.0.  Synthetic uniform random token ids and
random-init N(0, 0.02) weights.

    python bench.py --gpus 1 --steps 5 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29511 bench.py --gpus 8 --steps 5 --warmup 3
    python bench.py --impl reference ...   # the unmodified reference from baseline/_ref

Other named configurations through the same two arms: ``--parallel fsdp`` (N > 1: the reference's
FULL_SHARD wrapper against this package's sharded executor), ``--strategy dpo`` (a trainable policy
plus a frozen copy, 8 chosen/rejected pairs per GPU sharing a 512-token prompt with 512-token
responses, beta 0.1, one micro-batch per step), ``--serve 1`` (own arm, after the training
numbers: decode tokens/s and median time to first token of the continuous-batching server on the
same GPUs, tensor parallel when N > 1, reported under the ``serving`` key; on by default for the
8-GPU headline run, where it gives the TP=8 half of the metric).

Two numbers come out of the own arm: ``value`` — K steps timed on the device with CUDA
events, inputs already resident; and ``e2e`` — the same K steps through the public
``Trainer`` API, where every micro-batch is copied from pinned host memory and every
micro-batch loss is read back to the host.  Rank 0 prints one JSON line.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.abspath(__file__))
METRIC = "train_tokens_per_s_1B"
MODEL = dict(vocab_size=32000, dim=2048, n_layers=24, norm_eps=1e-5, dim_ffn=5632, tie_weight=True, max_len=2048,
             rope_theta=10000.0, n_heads=16, n_kv_heads=4)
SEQ, BPD, ACCUM = 2048, 4, 8
DPO_PROMPT, DPO_RESPONSE, DPO_PAIRS, DPO_BETA = 512, 512, 8, 0.1
LR, BETAS, WD, SMOOTH, CLIP = 3e-4, (0.9, 0.95), 0.01, 0.05, 1.0
SEED = 3407


class Workload:
    """Shape of one optimizer step for the chosen strategy (per GPU)."""

    def __init__(self, strategy: str, accum: int = 0):
        self.strategy = strategy
        if strategy == "dpo":
            self.seq, self.bpd, self.accum = DPO_PROMPT + DPO_RESPONSE, DPO_PAIRS, 1
            self.tokens_per_sample = 2 * self.seq           # chosen + rejected
            self.extra = {"beta": DPO_BETA}
            self.h2d_per_micro = self.bpd * (2 * self.seq * 8 + 2 * self.seq)   # two id tensors (int64), two masks (bool)
        else:
            self.seq, self.bpd, self.accum = SEQ, BPD, ACCUM
            if accum > 0:       # off-headline runs (e.g. 1: the gradient collective's share of a step is 8x larger)
                self.accum = accum
            self.tokens_per_sample = self.seq
            self.extra = {"label_smoothing": SMOOTH}
            self.h2d_per_micro = 2 * self.bpd * self.seq * 8                 # input and target ids (int64)

    def tokens_per_step(self, replicas: int) -> int:
        return self.accum * self.bpd * self.tokens_per_sample * replicas

    def dataset(self, n_samples: int, vocab: int, seed: int):
        return SyntheticPairs(n_samples, vocab, seed) if self.strategy == "dpo" else SyntheticTokens(n_samples, self.seq, vocab, seed)


# ----------------------------------------------------------------------------------------
# helpers shared by both arms
# ----------------------------------------------------------------------------------------
def env_rank():
    return int(os.environ.get("RANK", 0)), int(os.environ.get("LOCAL_RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device_index: int):
        self.device_index = device_index
        self.proc = None
        self.path = None

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "200",
                 "-i", str(self.device_index)], stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, smax, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        try:
            for line in open(self.path):
                parts = [p.strip() for p in line.split(",")]
                if len(parts) < 9:
                    continue
                try:
                    sm.append(float(parts[1]))
                    smax.append(float(parts[2]))
                except ValueError:
                    continue
                for name, val in zip(names, parts[5:9]):
                    if val.lower().startswith("active"):
                        reasons.add(name)
            os.unlink(self.path)
        except Exception:
            pass
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(smax) if smax else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def max_over_ranks(ms: float, device) -> float:
    if dist.is_initialized():
        t = torch.tensor([ms], dtype=torch.float64, device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())
    return ms


def barrier_sync():
    if dist.is_initialized():
        dist.barrier()
    torch.cuda.synchronize()


class SyntheticTokens(torch.utils.data.Dataset):
    """Uniform random token ids, generated once on the host (pinned by the DataLoader)."""

    def __init__(self, n_samples: int, seq: int, vocab: int, seed: int):
        g = torch.Generator().manual_seed(seed)
        self.data = torch.randint(0, vocab, (n_samples, seq + 1), generator=g, dtype=torch.long)

    def __len__(self):
        return self.data.shape[0]

    def __getitem__(self, i):
        row = self.data[i]
        return {"input_ids": row[:-1], "target_ids": row[1:]}


class SyntheticPairs(torch.utils.data.Dataset):
    """Chosen / rejected pairs sharing a prompt: uniform random ids, the loss covers the responses."""

    def __init__(self, n_samples: int, vocab: int, seed: int):
        g = torch.Generator().manual_seed(seed)
        prompt = torch.randint(0, vocab, (n_samples, DPO_PROMPT), generator=g, dtype=torch.long)
        self.chosen = torch.cat([prompt, torch.randint(0, vocab, (n_samples, DPO_RESPONSE), generator=g)], dim=1)
        self.rejected = torch.cat([prompt, torch.randint(0, vocab, (n_samples, DPO_RESPONSE), generator=g)], dim=1)
        self.mask = torch.cat([torch.zeros(DPO_PROMPT, dtype=torch.bool), torch.ones(DPO_RESPONSE, dtype=torch.bool)])

    def __len__(self):
        return self.chosen.shape[0]

    def __getitem__(self, i):
        return {"chosen": self.chosen[i], "rejected": self.rejected[i], "chosen_mask": self.mask, "rejected_mask": self.mask}


class StepTimer:
    """Trainer callback (both arms): times exactly ``steps`` optimizer steps after ``warmup``
    ones with CUDA events bracketed by barrier + synchronize."""

    def __init__(self, warmup: int, steps: int, accum: int, device_index: int, count_launches=None):
        self.first = warmup * accum
        self.last = (warmup + steps) * accum
        self.seen = 0
        self.ms = None
        self.launches = None
        self.clocks = None
        self._count = count_launches
        self._sampler = ClockSampler(device_index)
        self.final_loss = None

    def on_batch_end(self, context):
        self.final_loss = context.loss   # a float in the reference, a device scalar here; read after the run

    def on_batch_begin(self, context):
        if self.seen == self.first:
            barrier_sync()
            self._sampler.start()
            self._l0 = self._count() if self._count else 0
            self._e0 = torch.cuda.Event(enable_timing=True)
            self._e1 = torch.cuda.Event(enable_timing=True)
            self._e0.record()
        self.seen += 1

    def on_train_end(self, context):
        self._finish()

    def on_epoch_end(self, context):
        self._finish()

    def _finish(self):
        if self.ms is not None or self.seen < self.last:
            return
        self._e1.record()
        barrier_sync()
        self.ms = self._e0.elapsed_time(self._e1)
        if dist.is_initialized():  # max over ranks while the trainer's process group is alive
            t = torch.tensor([self.ms], dtype=torch.float64, device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            self.ms = float(t.item())
        self.launches = (self._count() - self._l0) if self._count else None
        self.clocks = self._sampler.stop()


def emit(payload: dict):
    if env_rank()[0] == 0:
        print(json.dumps(payload), flush=True)


def base_payload(args, ws: int, impl: str, wl: "Workload") -> dict:
    par = args.parallel if ws > 1 else "single"
    cfg = {"model": "1B decoder (24L, d2048, 16q/4kv heads, ffn5632, vocab32000, tied)",
           "global_batch": wl.bpd * wl.accum * ws, "micro_batch_per_gpu": wl.bpd, "grad_accum": wl.accum,
           "seq_len": wl.seq, "parallelism": (f"dp{ws}" if par == "ddp" else f"{par}{ws}") if ws > 1 else "single",
           "strategy": wl.strategy,
           "optimizer": "AdamW lr3e-4 betas(0.9,0.95) wd0.01 clip1.0" + (" label_smoothing0.05" if wl.strategy == "seq" else f" dpo beta{DPO_BETA}"),
           "l2": "no flush: weights (2.3 GB) + activations exceed the 126 MB L2 every step"}
    if wl.strategy == "dpo":
        cfg["pairs_per_gpu"] = wl.bpd
        cfg["prompt_len"], cfg["response_len"] = DPO_PROMPT, DPO_RESPONSE
    return {"metric": METRIC, "unit": "tokens/s", "n_gpus": ws, "steps": args.steps, "warmup": args.warmup,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "impl": impl, "config": cfg}


def strip_untimed_callbacks(trainer) -> None:
    """Both arms: the end-of-run checkpoint (2.3 GB of safetensors) and the progress bar are not part of a step."""
    trainer.callbacks = [cb for cb in trainer.callbacks
                         if type(cb).__name__ not in ("CheckpointCallback", "ProgressBarCallback")]


# ----------------------------------------------------------------------------------------
# own arm
# ----------------------------------------------------------------------------------------
def run_own(args):
    rank, local_rank, ws = env_rank()
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if ws > 1 and not dist.is_initialized():
        dist.init_process_group("nccl", device_id=device)
    sys.path.insert(0, ROOT)
    from khaosz_b200 import AutoRegressiveLM, AutoRegressiveLMConfig, TrainConfig
    from khaosz_b200.models.components.layers import Linear
    from khaosz_b200.ops import _lib, raise_on_device_error
    from khaosz_b200.parallel import ExecutorFactory
    from khaosz_b200.trainer import FusedAdamW, SchedulerFactory, StrategyFactory, Trainer

    cfg = AutoRegressiveLMConfig(**MODEL)
    wl = Workload(args.strategy, args.accum)
    mode = args.parallel if ws > 1 else "none"
    replicas = 1 if mode == "tp" else ws  # data-parallel replicas
    args.cuda_graph = bool(args.cuda_graph) if args.cuda_graph >= 0 else mode == "tp"
    steps_total = args.warmup + args.steps
    accum = wl.accum

    def model_fn():
        torch.manual_seed(SEED)
        model = AutoRegressiveLM(cfg)
        for m in model.modules():
            if isinstance(m, Linear):
                torch.nn.init.normal_(m.weight, mean=0.0, std=0.02)
        return model.to(dtype=torch.bfloat16)

    def optimizer_fn(model):
        return FusedAdamW(model.parameters(), lr=LR, betas=BETAS, weight_decay=WD)

    def scheduler_fn(opt):
        return SchedulerFactory.create(opt, "cosine", warmup_steps=1, lr_decay_steps=10_000)

    # ---- device-timed steps (inputs resident on the device; every step sees data it has not seen) ----
    model = model_fn().to(device)
    ex_extra = {"overlap_grad_reduce": bool(args.overlap)} if args.overlap >= 0 and mode in ("ddp", "fsdp", "fsdp_zero1") else {}
    executor = ExecutorFactory.create(mode, grad_accum_steps=accum, cuda_graph=args.cuda_graph, **ex_extra)
    opt = optimizer_fn(model)
    model, opt, _, sched = executor.prepare(model, opt, None, scheduler_fn(opt))
    strategy = StrategyFactory.create(wl.strategy, model, device, executor=executor, model_fn=model_fn, **wl.extra)
    data = wl.dataset(steps_total * accum * wl.bpd, MODEL["vocab_size"], SEED + (rank if replicas > 1 else 0))
    micro = []
    for i in range(steps_total * accum):
        rows = [data[i * wl.bpd + j] for j in range(wl.bpd)]
        micro.append({k: torch.stack([r[k] for r in rows]).to(device) for k in rows[0]})
    model.train()
    cursor = [0]

    def one_step():
        for _ in range(accum):
            batch = micro[cursor[0] % len(micro)]
            cursor[0] += 1
            with executor.accumulate(model):
                loss = executor.micro_step(strategy, batch)
                if executor.sync_gradients:
                    opt.fused_clip(CLIP)
                    opt.step()
                    opt.zero_grad()
                    sched.step()
        return loss

    for _ in range(args.warmup):
        one_step()
    barrier_sync()
    sampler = ClockSampler(local_rank)
    sampler.start()
    l0 = _lib.launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        loss = one_step()
    e1.record()
    barrier_sync()
    ms = max_over_ranks(e0.elapsed_time(e1), device)
    launches = _lib.launch_count() - l0
    clocks = sampler.stop()
    final_loss = float(loss)
    peak_alloc_gb = round(torch.cuda.max_memory_allocated(device) / 2 ** 30, 2)
    free_b, total_b = torch.cuda.mem_get_info(device)
    device_used_gb = round((total_b - free_b) / 2 ** 30, 2)   # allocator cache + symmetric memory + context
    raise_on_device_error()
    tokens = args.steps * wl.tokens_per_step(replicas)
    value = tokens / (ms / 1e3)
    del model, opt, sched, strategy, executor, micro, data
    torch.cuda.empty_cache()

    # ---- end to end through the public Trainer API ----
    e2e = None
    if not args.no_e2e:
        n_samples = steps_total * accum * wl.bpd * replicas
        dataset = wl.dataset(n_samples, MODEL["vocab_size"], SEED)
        timer = StepTimer(args.warmup, args.steps, accum, local_rank, _lib.launch_count)
        tmp = tempfile.mkdtemp(prefix="kb200_bench_")
        tc = TrainConfig(model_fn=model_fn, strategy=wl.strategy, dataset=dataset, optimizer_fn=optimizer_fn,
                         scheduler_fn=scheduler_fn, n_epoch=1, batch_per_device=wl.bpd, grad_accum_steps=accum,
                         max_grad_norm=CLIP, ckpt_dir=tmp, ckpt_interval=10 ** 9, log_dir=os.path.join(tmp, "logs"),
                         log_interval=accum, random_seed=SEED, num_workers=0, pin_memory=True, nprocs=ws,
                         backend="nccl", parallel_mode=mode, device_type="cuda",
                         executor_kwargs={"cuda_graph": args.cuda_graph, **ex_extra}, extra_kwargs=dict(wl.extra))

        trainer = Trainer(tc, callbacks=[timer])
        strip_untimed_callbacks(trainer)
        trainer.train()
        ms_e2e = timer.ms  # already the max over ranks
        e2e = {"value": tokens / (ms_e2e / 1e3), "unit": "tokens/s", "ms_per_step": ms_e2e / args.steps,
               "h2d_bytes_per_step": accum * wl.h2d_per_micro, "d2h_bytes_per_step": accum * 4,
               "final_loss": float(timer.final_loss) if timer.final_loss is not None else None,
               "api": "khaosz_b200.trainer.Trainer.train (DataLoader pin_memory -> H2D per micro-batch, "
                      "loss read back per micro-batch)"}

    payload = base_payload(args, ws, "khaosz_b200", wl)
    if mode == "tp":
        payload["scaling"] = "strong"
        payload["config"]["global_batch"] = wl.bpd * accum
    payload.update({"value": value, "ms_per_step": ms / args.steps, "clocks": clocks, "gpu_launches": launches,
                    "final_loss": final_loss, "peak_alloc_gb": peak_alloc_gb, "device_used_gb": device_used_gb})
    if e2e is not None:
        payload["e2e"] = e2e
    if dist.is_initialized():
        dist.destroy_process_group()
    serve = args.serve if args.serve >= 0 else int(ws == 8 and mode == "ddp" and args.strategy == "seq")
    if serve and rank == 0:
        # the other ranks are done and leave; this one frees its memory and runs the serving job as a child
        torch.cuda.empty_cache()
        payload["serving"] = run_serving_child(ws)
    emit(payload)


def run_serving_child(ws: int) -> dict:
    """Decode tokens/s and median time to first token of the continuous-batching server on the same
    GPUs (tensor parallel over all of them when N > 1): 256 Poisson arrivals at 64 requests/s, prompts
    uniform in [128, 2048] random ids, 256 greedy tokens each, 16-token KV pages, bf16.

    Runs as a child job (``khaosz_b200.cli.benchmark serve`` under its own launcher) after the training
    ranks have released the GPUs, with a hard time limit: whatever happens to it, the training numbers
    above are already measured and still get printed."""
    serve = ["-m", "khaosz_b200.cli.benchmark", "serve", "--preset", "1b", "--requests", "256", "--rate", "64",
             "--gen_length", "256", "--max_batch_size", "256", "--page_size", "16", "--budget_s", "150"]
    if ws > 1:
        port = str(int(os.environ.get("MASTER_PORT", "29500")) + 17)
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={ws}", "--master-addr",
               "127.0.0.1", "--master-port", port] + serve
    else:
        cmd = [sys.executable] + serve
    drop = ("RANK", "LOCAL_RANK", "WORLD_SIZE", "LOCAL_WORLD_SIZE", "GROUP_RANK", "GROUP_WORLD_SIZE", "ROLE_RANK",
            "ROLE_NAME", "ROLE_WORLD_SIZE", "MASTER_ADDR", "MASTER_PORT")
    env = {k: v for k, v in os.environ.items() if k not in drop and not k.startswith("TORCHELASTIC")}
    try:
        res = subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=420)
        rows = [line for line in res.stdout.splitlines() if line.startswith("{") and '"benchmark"' in line]
        if not rows:
            return {"unavailable": ("no result line; " + (res.stderr.strip().splitlines() or ["rc %d" % res.returncode])[-1])[:300]}
        row = json.loads(rows[-1])
        return {"decode_tokens_per_s": row.get("decode_tokens_per_s_busy"),
                "output_tokens_per_s_wall": row.get("output_tokens_per_s_wall"), "ttft_p50_s": row.get("ttft_p50_s"),
                "ttft_p99_s": row.get("ttft_p99_s"), "tensor_parallel": ws, "weights": "bf16",
                "requests": row.get("requests"), "arrival_rate_per_s": row.get("arrival_rate_per_s"),
                "generated_per_request": row.get("generated_per_request"), "page_size": 16,
                "cut_at_budget": row.get("cut_at_budget"),
                "clock": "host wall clock around the trace (requests arrive over seconds); decode_tokens_per_s counts the "
                         "time the decode loop was busy"}
    except subprocess.TimeoutExpired:
        return {"unavailable": "the serving job did not finish within its time limit"}
    except Exception as exc:   # the training numbers stand on their own
        return {"unavailable": f"{type(exc).__name__}: {exc}"[:300]}


# ----------------------------------------------------------------------------------------
# reference arm: the unmodified reference package installed under baseline/_ref
# ----------------------------------------------------------------------------------------
def _install_h5py_stub():
    """The reference imports h5py at module import; the wheel is not available offline.  The
    bench never touches HDF5, so an empty stand-in module satisfies the import."""
    try:
        import h5py  # noqa: F401
    except ImportError:
        import types

        stub = types.ModuleType("h5py")

        class _Missing:
            def __init__(self, *a, **k):
                raise ImportError("h5py is not installed (bench stub)")

        stub.File = _Missing
        sys.modules["h5py"] = stub


def run_reference(args):
    ref_root = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref_root, "astrai")):
        print(json.dumps({"impl": "reference", "unavailable": "baseline/_ref/astrai is not installed"}), flush=True)
        return
    rank, local_rank, ws = env_rank()
    try:
        _install_h5py_stub()
        sys.path.insert(0, ref_root)
        import astrai  # noqa: F401
        from astrai.config import AutoRegressiveLMConfig, TrainConfig
        from astrai.model import AutoRegressiveLM
        from astrai.model.components.linear import Linear
        from astrai.trainer import SchedulerFactory, Trainer
    except Exception as exc:  # pragma: no cover
        if rank == 0:
            print(json.dumps({"impl": "reference", "unavailable": f"import failed: {type(exc).__name__}: {exc}"[:300]}),
                  flush=True)
        return
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    cfg = AutoRegressiveLMConfig(**MODEL)
    wl = Workload(args.strategy, args.accum)
    steps_total = args.warmup + args.steps
    if ws > 1 and args.parallel not in ("ddp", "fsdp"):
        if rank == 0:
            print(json.dumps({"impl": "reference", "unavailable": f"the reference has no '{args.parallel}' executor "
                              "(its parallel_mode choices are none, ddp and fsdp)"}), flush=True)
        return

    def model_fn():
        torch.manual_seed(SEED)
        model = AutoRegressiveLM(cfg)
        for m in model.modules():
            if isinstance(m, Linear):
                torch.nn.init.normal_(m.weight, mean=0.0, std=0.02)
        return model.to(dtype=torch.bfloat16)

    def optimizer_fn(model):
        return torch.optim.AdamW(model.parameters(), fused=True, lr=LR, betas=BETAS, weight_decay=WD)

    def scheduler_fn(opt):
        return SchedulerFactory.create(opt, schedule_type="cosine", warmup_steps=1, lr_decay_steps=10_000)

    dataset = wl.dataset(steps_total * wl.accum * wl.bpd * ws, MODEL["vocab_size"], SEED)
    timer = StepTimer(args.warmup, args.steps, wl.accum, local_rank)
    tmp = tempfile.mkdtemp(prefix="ref_bench_")
    mode = args.parallel if ws > 1 else "none"
    ex_kwargs = {"gradient_as_bucket_view": True, "broadcast_buffers": False} if mode == "ddp" else {}
    tc = TrainConfig(model_fn=model_fn, strategy=wl.strategy, dataset=dataset, optimizer_fn=optimizer_fn,
                     scheduler_fn=scheduler_fn, n_epoch=1, batch_per_device=wl.bpd, grad_accum_steps=wl.accum,
                     max_grad_norm=CLIP, ckpt_dir=tmp, ckpt_interval=10 ** 9, log_dir=os.path.join(tmp, "logs"),
                     log_interval=wl.accum, random_seed=SEED, num_workers=0, pin_memory=True, nprocs=ws, backend="nccl",
                     parallel_mode=mode, device_type="cuda", executor_kwargs=ex_kwargs, extra_kwargs=dict(wl.extra))
    trainer = Trainer(tc, callbacks=[timer])
    strip_untimed_callbacks(trainer)
    try:
        trainer.train()
    except Exception as exc:
        if rank == 0:
            print(json.dumps({"impl": "reference", "unavailable": f"run failed: {type(exc).__name__}: {exc}"[:300]}),
                  flush=True)
        return
    ms = timer.ms  # already the max over ranks
    tokens = args.steps * wl.tokens_per_step(ws)
    payload = base_payload(args, ws, "reference", wl)
    val = tokens / (ms / 1e3)
    payload.update({"value": val, "ms_per_step": ms / args.steps, "clocks": timer.clocks, "gpu_launches": None,
                    "final_loss": float(timer.final_loss) if timer.final_loss is not None else None,
                    "e2e": {"value": val, "unit": "tokens/s", "h2d_bytes_per_step": wl.accum * wl.h2d_per_micro,
                            "d2h_bytes_per_step": wl.accum * 4,
                            "final_loss": float(timer.final_loss) if timer.final_loss is not None else None,
                            "api": "astrai.trainer.Trainer.train (the reference's only training path: H2D per "
                                   "micro-batch and loss.item() per micro-batch are inside it)"}})
    emit(payload)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="khaosz_b200", choices=["khaosz_b200", "own", "reference"])
    ap.add_argument("--no-e2e", dest="no_e2e", action="store_true")
    ap.add_argument("--cuda-graph", dest="cuda_graph", type=int, default=-1,
                    help="own arm: forward+backward of a micro-batch as a replayed CUDA graph (default: on for tp)")
    ap.add_argument("--parallel", default="ddp", choices=["ddp", "fsdp", "fsdp_block", "fsdp_zero1", "fsdp_full", "tp"],
                    help="own arm, N > 1: data parallel (default), sharded data parallel, or tensor parallel "
                         "(tp: every rank reads the same batches, total work is fixed -> strong scaling)")
    ap.add_argument("--strategy", default="seq", choices=["seq", "dpo"],
                    help="seq: next-token pre-training (the headline); dpo: policy + frozen copy on chosen/rejected pairs")
    ap.add_argument("--accum", type=int, default=0,
                    help="micro-batches per optimizer step of the seq strategy (default: the headline's 8)")
    ap.add_argument("--overlap", type=int, default=-1,
                    help="own arm, ddp / fsdp: 1 hands gradient buckets to the reduce kernels during the backward pass")
    ap.add_argument("--serve", type=int, default=-1,
                    help="own arm: 1 appends decode tokens/s and median time to first token of the server on the same "
                         "GPUs (a child job after the training numbers); default: only for the 8-GPU headline run")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 0)
    ws = env_rank()[2]
    if args.gpus > 1 and ws == 1:
        # convenience: re-launch under torchrun when called directly with --gpus N
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={args.gpus}",
               "--master-addr", "127.0.0.1", "--master-port", os.environ.get("MASTER_PORT", "29533"),
               os.path.abspath(__file__)] + sys.argv[1:]
        sys.exit(subprocess.call(cmd))
    if not torch.cuda.is_available():
        print(json.dumps({"impl": args.impl, "unavailable": "no CUDA device visible"}), flush=True)
        return
    if args.impl == "reference":
        run_reference(args)
    else:
        run_own(args)


if __name__ == "__main__":
    main()
