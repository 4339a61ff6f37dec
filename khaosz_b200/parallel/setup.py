"""Process launch and process-group lifecycle (one process per GPU).

API parity with ``astrai/parallel/setup.py:12-232``: ``spawn_parallel_fn`` runs ``func`` on
``world_size`` ranks — in-process when ``world_size == 1``, under the ranks an external
launcher (torchrun / torchelastic / SLURM) already created when its environment variables
are present, otherwise as locally spawned children that are torn down together if any of
them fails.  ``setup_parallel`` exports ``MASTER_*``, ``LOCAL_RANK``, ``WORLD_SIZE`` and
``LOCAL_DEVICE`` and owns ``init_process_group`` / ``destroy_process_group``.

Unlike the reference a CUDA ``device_type`` degrades to CPU when no GPU is visible (so gloo
ranks work on a CPU-only host), ``KHAOSZ_B200_PG_TIMEOUT_S`` shortens the process-group timeout,
and a rank that unwinds an exception leaves without the collective tear-down so that the
launcher can stop the others.  The symmetric-memory rendezvous of the in-kernel collectives
runs over the same process group (``khaosz_b200.parallel.comm``).
"""

from __future__ import annotations

import contextlib
import functools
import os
from typing import Callable

import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def get_world_size() -> int:
    return dist.get_world_size() if dist.is_available() and dist.is_initialized() else 1


def get_rank() -> int:
    return dist.get_rank() if dist.is_available() and dist.is_initialized() else 0


def get_current_device() -> str:
    """Device string of this rank (``cuda:3`` / ``cpu``) as exported by ``setup_parallel``."""
    return os.environ.get("LOCAL_DEVICE", "cuda:0" if torch.cuda.is_available() else "cpu")


def _resolve_device(device_type: str, local_rank: int) -> torch.device:
    if device_type == "cuda" and not torch.cuda.is_available():
        return torch.device("cpu")
    if device_type == "cpu":
        return torch.device("cpu")
    return torch.device(device_type, local_rank)


@contextlib.contextmanager
def setup_parallel(rank: int, world_size: int, local_rank: int, backend: str = "nccl",
                   master_addr: str = "localhost", master_port: str = "29500", device_type: str = "cuda"):
    device = _resolve_device(device_type, local_rank)
    if dist.is_available() and dist.is_initialized():
        # an outer scope owns the group; still export this rank's device
        os.environ["LOCAL_RANK"] = str(local_rank)
        os.environ["LOCAL_DEVICE"] = str(device)
        if device.type == "cuda":
            torch.cuda.set_device(device)
        yield dist.group.WORLD
        return
    os.environ["LOCAL_RANK"] = str(local_rank)
    os.environ["WORLD_SIZE"] = str(max(world_size, 1))
    os.environ["LOCAL_DEVICE"] = str(device)
    if device.type == "cuda":
        torch.cuda.set_device(device)
    if world_size <= 1:
        yield None
        return
    os.environ["MASTER_ADDR"] = master_addr
    os.environ["MASTER_PORT"] = str(master_port)
    kwargs = {}
    if backend == "nccl" and device.type == "cuda":
        kwargs["device_id"] = device
    if os.environ.get("KHAOSZ_B200_PG_TIMEOUT_S"):
        import datetime

        kwargs["timeout"] = datetime.timedelta(seconds=float(os.environ["KHAOSZ_B200_PG_TIMEOUT_S"]))
    dist.init_process_group(backend=backend, rank=rank, world_size=world_size, **kwargs)
    failed = False
    try:
        yield dist.group.WORLD
    except BaseException:
        failed = True
        raise
    finally:
        # A rank that is unwinding an exception must not wait for its peers in a collective
        # tear-down: it has to exit so that the launcher sees the failure and stops the others.
        if not failed and dist.is_initialized():
            try:
                # leave together: a rank that closes its transport while a peer still has traffic
                # in flight (gloo) aborts that peer
                dist.barrier()
            except Exception:  # a peer that is already gone must not turn a finished run into a failure
                pass
            dist.destroy_process_group()


def only_on_rank(rank: int, sync: bool = False):
    """Decorator: run the function on one rank only (others return None); ``sync`` adds a
    barrier afterwards."""

    def deco(fn):
        @functools.wraps(fn)
        def wrapped(*args, **kwargs):
            result = fn(*args, **kwargs) if get_rank() == rank else None
            if sync and dist.is_available() and dist.is_initialized():
                dist.barrier()
            return result

        return wrapped

    return deco


def _rank_entry(rank: int, world_size: int, backend: str, master_addr: str, master_port: str, device_type: str,
                func: Callable, kwargs: dict) -> None:
    with setup_parallel(rank, world_size, rank, backend, master_addr, master_port, device_type):
        func(**kwargs)


def detect_launcher() -> str:
    """``torchelastic`` | ``torchrun`` | ``external`` (RANK/WORLD_SIZE preset) | ``local``."""
    if dist.is_available() and dist.is_torchelastic_launched():
        return "torchelastic"
    if "LOCAL_WORLD_SIZE" in os.environ:
        return "torchrun"
    if "RANK" in os.environ and "WORLD_SIZE" in os.environ:
        return "external"
    return "local"


def _launch_under_external(func, backend, master_addr, master_port, device_type, kwargs) -> None:
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local_rank = int(os.environ.get("LOCAL_RANK", rank))
    with setup_parallel(rank, world, local_rank, backend, os.environ.get("MASTER_ADDR", master_addr),
                        os.environ.get("MASTER_PORT", master_port), device_type):
        func(**kwargs)


def _launch_local(func, world_size, backend, master_addr, master_port, device_type, start_method, kwargs) -> None:
    args = (world_size, backend, master_addr, master_port, device_type, func, kwargs)
    if world_size <= 1:
        _rank_entry(0, *args)
        return
    ctx = mp.start_processes(_rank_entry, args=args, nprocs=world_size, start_method=start_method, join=False)
    try:
        while not ctx.join(timeout=5):
            pass
    except BaseException:
        for proc in ctx.processes:
            if proc.is_alive():
                proc.terminate()
        for proc in ctx.processes:
            proc.join(timeout=10)
        raise


def spawn_parallel_fn(func: Callable, world_size: int, backend: str = "nccl", master_addr: str = "localhost",
                      master_port: str = "29500", device_type: str = "cuda", start_method: str = "spawn",
                      **kwargs) -> None:
    if detect_launcher() == "local":
        _launch_local(func, world_size, backend, master_addr, master_port, device_type, start_method, kwargs)
    else:
        _launch_under_external(func, backend, master_addr, master_port, device_type, kwargs)
