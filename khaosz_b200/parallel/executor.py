"""Execution strategies behind the trainer: ``none``, ``ddp``, ``fsdp`` and ``tp``.

The contract is the reference's (``astrai/parallel/executor.py:82-137``)::

    model, optimizer, dataloader, scheduler = executor.prepare(model, optimizer, dataloader, scheduler)
    with executor.accumulate(model):
        loss = ...; executor.backward(loss / executor.grad_accum_steps)
        if executor.sync_gradients: optimizer.step(); optimizer.zero_grad(); scheduler.step()
    full_state_dict = executor.unwrap_model(model)

but the machinery is rebuilt: instead of wrapping the model in torch DDP / FSDP, an executor
owns *flat* parameter and gradient buffers (``khaosz_b200.utils.FlatParameters``).  Weight
gradients are accumulated into the flat gradient buffer by the GEMM epilogues, the gradient
collective runs once per optimizer step over that buffer (hand-written NVLink kernels on
CUDA, ``torch.distributed`` on CPU/gloo), and a ``FusedAdamW`` optimizer updates the whole
model in one launch.  ``ddp`` replicates parameters; ``fsdp`` shards gradients, optimizer
state and the update (each rank owns a contiguous slice, updated parameters are
all-gathered); ``tp`` is described in ``khaosz_b200.parallel.tensor_parallel``.
"""

from __future__ import annotations

import contextlib
import logging
import os
from typing import Any, Dict, Optional, Tuple

import torch
import torch.distributed as dist
import torch.nn as nn

from ..factory import BaseFactory
from ..utils.flat_params import FlatParameters
from .setup import get_rank, get_world_size

log = logging.getLogger(__name__)


class GradientState:
    """Counts micro-steps globally; gradients are synchronised every ``num_steps``-th one."""

    def __init__(self, grad_accum_steps: int = 1):
        self.num_steps = max(int(grad_accum_steps), 1)
        self._step = 0
        self._sync_gradients = True

    @property
    def sync_gradients(self) -> bool:
        return self._sync_gradients

    def _do_sync(self) -> None:
        self._step += 1
        self._sync_gradients = self._step % self.num_steps == 0


class AccumOptimizer:
    """Optimizer facade that only acts on synchronisation steps.  ``zero_grad`` keeps
    ``param.grad`` aliased to the flat gradient buffer when the executor owns one."""

    def __init__(self, optimizer, gradient_state: GradientState, flat: Optional[FlatParameters] = None,
                 after_step=None):
        self.optimizer = optimizer
        self.gradient_state = gradient_state
        self.flat = flat
        self._after_step = after_step

    def step(self, closure=None):
        if self.gradient_state.sync_gradients:
            self.optimizer.step(closure) if closure is not None else self.optimizer.step()
            if self._after_step is not None:
                self._after_step()

    def zero_grad(self, *args, **kwargs):
        if not self.gradient_state.sync_gradients:
            return
        if self.flat is not None and self.flat.grad is not None:
            self.flat.zero_grad()
        else:
            self.optimizer.zero_grad(*args, **kwargs)

    @property
    def param_groups(self):
        return self.optimizer.param_groups

    def state_dict(self):
        return self.optimizer.state_dict()

    def load_state_dict(self, state):
        self.optimizer.load_state_dict(state)

    def __getattr__(self, name):  # fused_clip, flat hooks, ...
        return getattr(self.optimizer, name)


class RankStateOptimizer(AccumOptimizer):
    """Facade for executors whose parameters differ from rank to rank (tensor parallel, fully
    sharded): ``state_dict`` is collective and returns one optimizer state per rank of the group, so
    that the single checkpoint rank 0 writes can restore every rank; ``load_state_dict`` picks this
    rank's entry (a plain state dict is loaded as is)."""

    def __init__(self, optimizer, gradient_state, flat=None, after_step=None, group=None, model=None):
        super().__init__(optimizer, gradient_state, flat, after_step)
        self.group = group
        self.model = model   # a model with gather_named / scatter_named makes the state portable

    def _layout(self):
        if not (dist.is_available() and dist.is_initialized()):
            return 0, 1
        return dist.get_rank(self.group), dist.get_world_size(self.group)

    def _local_params(self):
        return [p for g in self.optimizer.param_groups for p in g["params"]]

    def _portable(self, mine) -> bool:
        st = mine.get("state", {})
        return (self.model is not None and hasattr(self.model, "gather_named") and len(st) == len(self._local_params())
                and all(isinstance(v, dict) and set(v) >= {"step", "exp_avg", "exp_avg_sq"} for v in st.values()))

    def state_dict(self):
        mine = self.optimizer.state_dict()
        rank, ws = self._layout()
        if ws == 1:
            return mine
        if self._portable(mine):
            # Adam-style moments: assemble them to the dense model's parameter order, i.e. the same
            # optimizer.pt layout a single-process or data-parallel run writes
            params = self._local_params()
            by_id = {id(p): mine["state"][i] for i, p in enumerate(params)}
            full = {}
            for key in ("exp_avg", "exp_avg_sq"):
                full[key] = self.model.gather_named(lambda p, k=key: by_id[id(p)][k].to(p.device))
            step = next(iter(mine["state"].values()))["step"]
            state = {i: {"step": step, "exp_avg": full["exp_avg"][n].cpu(), "exp_avg_sq": full["exp_avg_sq"][n].cpu()}
                     for i, n in enumerate(self.model.dense_names)}
            group = {k: v for k, v in mine["param_groups"][0].items() if k != "params"}
            group["params"] = list(range(len(self.model.dense_names)))
            return {"state": state, "param_groups": [group]}
        states = [None] * ws
        dist.all_gather_object(states, mine, group=self.group)
        return {"per_rank": states}

    def load_state_dict(self, state):
        if (isinstance(state, dict) and "per_rank" not in state and self.model is not None
                and hasattr(self.model, "scatter_named") and self._layout()[1] > 1
                and len(state.get("state", {})) == len(getattr(self.model, "dense_names", ()))):
            names = self.model.dense_names
            get = lambda i: state["state"].get(i) or state["state"].get(str(i))
            params = self._local_params()
            local = {}
            for key in ("exp_avg", "exp_avg_sq"):
                sliced = self.model.scatter_named({n: get(i)[key] for i, n in enumerate(names)})
                for j, p in enumerate(params):
                    local.setdefault(j, {"step": get(0)["step"]})[key] = sliced[id(p)].contiguous()
            group = dict(state["param_groups"][0])
            group["params"] = list(range(len(params)))
            self.optimizer.load_state_dict({"state": local, "param_groups": [group]})
            return
        if isinstance(state, dict) and "per_rank" in state:
            rank, ws = self._layout()
            if len(state["per_rank"]) != ws:
                raise ValueError(f"checkpoint holds optimizer states of {len(state['per_rank'])} ranks, this group has {ws}")
            state = state["per_rank"][rank]
        self.optimizer.load_state_dict(state)


class AccumScheduler:
    def __init__(self, scheduler, gradient_state: GradientState):
        self.scheduler = scheduler
        self.gradient_state = gradient_state

    def step(self):
        if self.gradient_state.sync_gradients:
            self.scheduler.step()

    def state_dict(self):
        return self.scheduler.state_dict()

    def load_state_dict(self, state):
        self.scheduler.load_state_dict(state)

    def get_last_lr(self):
        return self.scheduler.get_last_lr()


class _GraphedMicroStep:
    """Forward + backward of one micro-batch as a CUDA graph per batch signature.

    The first two micro-batches of a signature run with plain launches (lazy allocations, symmetric
    buffers, kernel attributes); the third is captured over static input buffers; from then on a
    micro-batch is two small copies and one graph launch.  A step is a few thousand launches of
    kernels that take 10-100 us each, so without the graph the host thread is the bottleneck once
    the per-GPU work shrinks (tensor parallelism)."""

    WARMUP = 2

    def __init__(self, executor: "BaseExecutor"):
        self.executor = executor
        self.entries: Dict[Any, Dict[str, Any]] = {}
        self.disabled = False

    @staticmethod
    def _signature(batch: Dict[str, Any]):
        return tuple(sorted((k, tuple(v.shape), str(v.dtype)) for k, v in batch.items() if torch.is_tensor(v)))

    def __call__(self, strategy, batch: Dict[str, Any], scale: float) -> torch.Tensor:
        ex = self.executor
        key = self._signature(batch)
        entry = self.entries.setdefault(key, {"uses": 0})
        entry["uses"] += 1
        if self.disabled or entry["uses"] <= self.WARMUP:
            loss = strategy(batch)
            ex._backward_only(loss * scale)
            return loss.detach()
        device = strategy.device
        if "graph" not in entry:
            static = {k: (torch.empty_like(v, device=device) if torch.is_tensor(v) else v) for k, v in batch.items()}
            for k, v in batch.items():
                if torch.is_tensor(v):
                    static[k].copy_(v, non_blocking=True)
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            from ..ops import _lib

            before = _lib.launch_count()
            try:
                with torch.cuda.graph(graph, capture_error_mode="thread_local"):
                    loss = strategy(static)
                    ex._backward_only(loss * scale)
                    out = loss.detach()
            except Exception as exc:  # something in the step cannot be captured: keep plain launches
                log.warning("CUDA graph capture of the micro-step failed (%s); running without graphs", exc)
                self.disabled = True
                torch.cuda.synchronize()
                loss = strategy(batch)
                ex._backward_only(loss * scale)
                return loss.detach()
            # kernel-library launches recorded in the graph: every replay issues them again
            entry.update(graph=graph, static=static, loss=out, launches=_lib.launch_count() - before)
            _lib.add_launches(-entry["launches"])  # the recording itself launched nothing
            # Recording takes seconds and differs per rank; kernels that wait for their peers have a
            # bounded patience, so the ranks line up on the host before the first replay.
            if dist.is_available() and dist.is_initialized():
                torch.cuda.synchronize()
                dist.barrier()
        else:
            for k, v in batch.items():
                if torch.is_tensor(v):
                    entry["static"][k].copy_(v, non_blocking=True)
        entry["graph"].replay()
        if entry.get("launches"):
            from ..ops import _lib

            _lib.add_launches(entry["launches"])
        return entry["loss"].clone()


def _wants_flat(model: nn.Module) -> bool:
    params = list(model.parameters())
    return bool(params) and all(p.is_cuda and p.dtype == torch.bfloat16 for p in params)


class BaseExecutor:
    flatten_on_cuda = True

    def __init__(self, grad_accum_steps: int = 1, fp8: bool = False, cuda_graph: bool = False):
        self.gradient_state = GradientState(grad_accum_steps)
        self.flat: Optional[FlatParameters] = None
        self.fp8 = bool(fp8)
        self._graphed = _GraphedMicroStep(self) if cuda_graph and torch.cuda.is_available() else None
        if self.fp8:
            # forward GEMMs of the local linear layers in block-scaled fp8 (bf16 master weights); fp8="dgrad"
            # (or KHAOSZ_B200_FP8_DGRAD=1) runs the input-gradient GEMMs in fp8 as well
            from ..ops.functional import set_fp8_linear

            set_fp8_linear(True, dgrad=fp8 == "dgrad" or os.environ.get("KHAOSZ_B200_FP8_DGRAD", "0") == "1")

    # -- preparation ------------------------------------------------------------------------
    def prepare(self, model: nn.Module, optimizer=None, dataloader=None, scheduler=None) -> Tuple[Any, Any, Any, Any]:
        model = self._prepare_model(model)
        if optimizer is not None:
            if self.flat is not None and hasattr(optimizer, "attach_flat"):
                optimizer.attach_flat(self.flat)
            optimizer = AccumOptimizer(optimizer, self.gradient_state, self.flat, self._after_optimizer_step)
        if scheduler is not None:
            scheduler = AccumScheduler(scheduler, self.gradient_state)
        return model, optimizer, dataloader, scheduler

    def _prepare_model(self, model: nn.Module) -> nn.Module:
        if self.flatten_on_cuda and _wants_flat(model):
            self.flat = FlatParameters(model, with_grad=True)
        return model

    def _after_optimizer_step(self) -> None:
        """Hook for sharded executors (parameter all-gather)."""

    # -- the loop ---------------------------------------------------------------------------
    def _no_sync(self, model: nn.Module):
        return contextlib.nullcontext()

    def _begin_micro_step(self, final: bool) -> None:
        """``final``: this micro-batch ends the accumulation window (its gradients get reduced)."""
        reducer = getattr(self, "_reducer", None)
        if reducer is not None and getattr(self, "_fused", False) and hasattr(reducer, "begin_window"):
            reducer.begin_window(final)

    @contextlib.contextmanager
    def accumulate(self, model: nn.Module):
        self.gradient_state._do_sync()
        self._begin_micro_step(self.gradient_state.sync_gradients)
        ctx = contextlib.nullcontext() if self.gradient_state.sync_gradients else self._no_sync(model)
        with ctx:
            yield

    def backward(self, loss: torch.Tensor) -> None:
        self._backward_only(loss)
        if self.gradient_state.sync_gradients:
            self._sync_gradients()

    def _backward_only(self, loss: torch.Tensor) -> None:
        loss.backward()

    def micro_step(self, strategy, batch) -> torch.Tensor:
        """``loss = strategy(batch); backward(loss / grad_accum_steps)`` inside ``accumulate``;
        returns the detached loss.  With ``cuda_graph=True`` the pair runs as a replayed CUDA graph."""
        scale = 1.0 / self.gradient_state.num_steps
        if self._graphed is None:
            loss = strategy(batch)
            self.backward(loss * scale)
            return loss.detach()
        loss = self._graphed(strategy, batch, scale)
        if self.gradient_state.sync_gradients:
            self._sync_gradients()
        return loss

    def _sync_gradients(self) -> None:
        """Cross-rank gradient reduction on synchronisation steps."""

    def unwrap_model(self, model: nn.Module) -> Dict[str, torch.Tensor]:
        return model.state_dict()

    def grad_norm_sq_extra(self) -> Optional[torch.Tensor]:
        """Sharded executors return a device scalar with the *global* squared gradient norm."""
        return None

    @property
    def use_distributed(self) -> bool:
        return get_world_size() > 1

    @property
    def sync_gradients(self) -> bool:
        return self.gradient_state.sync_gradients

    @property
    def grad_accum_steps(self) -> int:
        return self.gradient_state.num_steps


class ExecutorFactory(BaseFactory[BaseExecutor]):
    pass


@ExecutorFactory.register("none")
class NoneExecutor(BaseExecutor):
    """Single process."""


def _broadcast_parameters(model: nn.Module, flat: Optional[FlatParameters]) -> None:
    if get_world_size() <= 1:
        return
    if flat is not None:
        dist.broadcast(flat.data, src=0)
        return
    for t in list(model.parameters()) + list(model.buffers()):
        dist.broadcast(t.data, src=0)


@ExecutorFactory.register("ddp")
class DDPExecutor(BaseExecutor):
    """Data parallel with replicated parameters.

    Works on CPU/gloo as well as CUDA/NCCL (the reference's wrapper cannot wrap a CPU model,
    ``astrai/parallel/executor.py:181-193``).  The torch-DDP keyword arguments of the
    reference are accepted for compatibility.  With ``overlap_grad_reduce=True`` the gradients leave
    in ``bucket_cap_mb`` buckets while the backward pass of the window's last micro-batch is still
    running (``khaosz_b200.parallel.comm.GradReducer``); by default they are reduced in one launch
    after it, which measured faster in every configuration tried (the reduction is a few milliseconds).
    """

    def __init__(self, grad_accum_steps: int = 1, find_unused_parameters: bool = False, bucket_cap_mb: int = 25,
                 gradient_as_bucket_view: bool = True, broadcast_buffers: bool = False, static_graph: bool = False,
                 init_sync: bool = True, comm: str = "auto", fp8: bool = False, cuda_graph: bool = False,
                 overlap_grad_reduce: Optional[bool] = None, **_ignored):
        super().__init__(grad_accum_steps, fp8, cuda_graph)
        self.bucket_cap_mb = bucket_cap_mb
        self.overlap_grad_reduce = overlap_grad_reduce   # None: KHAOSZ_B200_DDP_OVERLAP decides (default off)
        self.init_sync = init_sync
        self.comm = comm  # "auto" | "nccl" | "kernel"
        self._reducer = None

    def _prepare_model(self, model: nn.Module) -> nn.Module:
        params = list(model.parameters())
        same = len({(p.dtype, p.device) for p in params}) == 1
        if same:
            self.flat = FlatParameters(model, with_grad=True, pad_to=8 * max(get_world_size(), 1))
        self._model = model
        if self.flat is not None and self.flat.data.is_cuda and get_world_size() > 1 and self.comm != "nccl":
            from .comm import GradReducer

            self._reducer = GradReducer.create(self.flat, mode="allreduce", bucket_cap_mb=self.bucket_cap_mb,
                                               overlap=self.overlap_grad_reduce)
        if self.init_sync:
            if self._reducer is not None and self.flat.numel % 8 == 0:
                # rank 0's parameters to everybody through the NVLink broadcast kernel (one pass of
                # multimem / peer stores over the symmetric parameter buffer)
                from .comm import broadcast_

                broadcast_(self._reducer.params, self._reducer.ctrl, root=0, use_multicast=self._reducer.use_multicast)
                for t in model.buffers():
                    dist.broadcast(t.data, src=0)
            else:
                _broadcast_parameters(model, self.flat)
        return model

    def _sync_gradients(self) -> None:
        ws = get_world_size()
        if ws <= 1:
            return
        if self._reducer is not None:
            if not getattr(self, "_fused", False):
                self._reducer.allreduce_grads()  # the optimizer cannot fuse: kernel all-reduce only
            return
        if self.flat is not None:
            dist.all_reduce(self.flat.grad)
            self.flat.grad.div_(ws)
            return
        for p in self._model.parameters():
            if p.grad is not None:
                dist.all_reduce(p.grad)
                p.grad.div_(ws)

    def prepare(self, model, optimizer=None, dataloader=None, scheduler=None):
        model = self._prepare_model(model)
        self._fused = False
        if optimizer is not None:
            if self._reducer is not None and hasattr(optimizer, "attach_reducer"):
                optimizer.attach_flat(self.flat, allocate=False)
                if getattr(optimizer, "_flat", None) is not None:
                    optimizer.attach_reducer(self._reducer)
                    self._fused = True
                    self._reducer.install_hooks(model)   # buckets leave while the backward pass still runs
            elif self.flat is not None and hasattr(optimizer, "attach_flat"):
                optimizer.attach_flat(self.flat)
            optimizer = AccumOptimizer(optimizer, self.gradient_state, self.flat, self._after_optimizer_step)
        if scheduler is not None:
            scheduler = AccumScheduler(scheduler, self.gradient_state)
        return model, optimizer, dataloader, scheduler


def _why_not_block_sharded(model: nn.Module, optimizer, cuda_graph: bool) -> Optional[str]:
    """Reason why the block-granular full shard cannot take this model / optimizer (None: it can)."""
    if not isinstance(getattr(model, "layers", None), (nn.ModuleList, list, tuple)) or len(model.layers) == 0:
        return f"{type(model).__name__} has no `layers` list to shard by"
    params = list(model.parameters())
    if not params or not all(p.requires_grad for p in params):
        return "the model has frozen parameters (adapters)"
    if any(p.dtype != params[0].dtype or p.device != params[0].device for p in params):
        return "the parameters do not share one dtype and device"
    if optimizer is not None and (not hasattr(optimizer, "attach_flat") or len(optimizer.param_groups) != 1):
        return f"{type(optimizer).__name__} keeps per-parameter state (only the fused flat AdamW is sharded)"
    if cuda_graph:
        return "the micro-step is to be captured as a CUDA graph"
    if params[0].is_cuda and get_world_size() > 1:
        from ..ops import _lib

        if params[0].dtype != torch.bfloat16 or not _lib.has("kb_unit_reduce_bf16") or get_world_size() > 8:
            return "the collective kernels need bf16 parameters and at most 8 ranks"
    return None


@ExecutorFactory.register("fsdp")
class FSDPExecutor(BaseExecutor):
    """Fully sharded data parallel.

    ``shard_parameters=True`` (mode ``fsdp_block``; the default of ``fsdp`` wherever it applies): every
    decoder block's parameters, gradients and AdamW moments exist as one ``1 / ws`` piece per rank
    (``khaosz_b200.parallel.unit_shard``).  A block's weights are gathered into one of two reusable
    images before its forward and again before its backward, by the copy engine, while the previous
    block computes; its gradients are reduce-scattered by a kernel on a side stream while the next
    block's backward runs.  Modules, names and kernels are those of the dense model.  Embedding, final
    norm and an untied output layer stay replicated (one all-reduce of their gradients per step).  This is
    the memory behaviour of the reference's ``ShardingStrategy.FULL_SHARD`` wrapper
    (``astrai/parallel/executor.py:223-272``).

    ``shard_parameters=False`` (mode ``fsdp_zero1``; also what ``fsdp`` falls back to, with a warning, for
    models with frozen parameters, optimizers other than the fused AdamW or a captured micro-step):
    whole parameters and gradients stay resident; every rank owns the contiguous slice
    ``[rank * n / ws, (rank + 1) * n / ws)`` of the flat parameter vector, gradients are
    reduce-scattered to their owner, optimizer state exists for the owned slice only and the owner
    updates it; updated parameters are all-gathered before the next forward.

    ``unwrap_model`` returns the full (unsharded) state dict on every rank and the optimizer's
    ``state_dict`` the dense layout, as the reference's ``FULL_STATE_DICT`` gather does
    (``astrai/parallel/executor.py:263-272``).
    """

    default_shard_parameters: Optional[bool] = None     # None: where it applies

    def __init__(self, grad_accum_steps: int = 1, comm: str = "auto", fp8: bool = False, cuda_graph: bool = False,
                 bucket_cap_mb: int = 25, overlap_grad_reduce: Optional[bool] = None,
                 shard_parameters: Optional[bool] = None, prefetch: bool = True, **_ignored):
        super().__init__(grad_accum_steps, fp8, cuda_graph)
        self.comm = comm
        self.bucket_cap_mb = bucket_cap_mb
        self.overlap_grad_reduce = overlap_grad_reduce
        self.shard_parameters = self.default_shard_parameters if shard_parameters is None else shard_parameters
        self.prefetch = prefetch
        self.shard: Optional[Tuple[int, int]] = None
        self._reducer = None
        self.units = None
        self._wants_graph = bool(cuda_graph)

    def _block_sharded(self, model: nn.Module, optimizer) -> bool:
        want = self.shard_parameters
        if want is None:
            want = os.environ.get("KHAOSZ_B200_FSDP_SHARD_PARAMS", "1") != "0"
        if not want:
            return False
        why = _why_not_block_sharded(model, optimizer, self._wants_graph)
        if why is None:
            return True
        if self.shard_parameters:
            raise NotImplementedError(f"fsdp_block: {why}; use fsdp_zero1 or ddp")
        log.warning("fsdp: %s; whole parameters stay resident on every rank, the optimizer state and the update "
                    "are sharded (fsdp_zero1)", why)
        return False

    def _prepare_model(self, model: nn.Module) -> nn.Module:
        ws = get_world_size()
        self.flat = FlatParameters(model, with_grad=True, pad_to=8 * max(ws, 1))
        _broadcast_parameters(model, self.flat)
        n = self.flat.numel // max(ws, 1)
        self.shard = (get_rank() * n, n)
        self._model = model
        if self.flat.data.is_cuda and ws > 1 and self.comm != "nccl":
            from .comm import GradReducer

            self._reducer = GradReducer.create(self.flat, mode="reducescatter", bucket_cap_mb=self.bucket_cap_mb,
                                               overlap=self.overlap_grad_reduce)
        return model

    def _prepare_units(self, model: nn.Module, optimizer):
        from .unit_shard import ShardedUnits

        _broadcast_parameters(model, None)
        self._graphed = None        # the side streams' events are not captured
        self.units = ShardedUnits(model, prefetch=self.prefetch)
        self.flat = self.units.flat
        self._model = model
        if optimizer is not None:
            optimizer.attach_flat(self.flat, shard=(0, self.units.local_numel))
            if getattr(optimizer, "_flat", None) is None:
                raise NotImplementedError("fsdp: the optimizer has to cover exactly the model's parameters")
            optimizer.set_layout(self.units.owned_ranges)
            optimizer.set_norm_fn(self.units.grad_norm_sq)
            optimizer = AccumOptimizer(optimizer, self.gradient_state, self.flat, self._after_optimizer_step)
        return model, optimizer

    def prepare(self, model, optimizer=None, dataloader=None, scheduler=None):
        if self._block_sharded(model, optimizer):
            model, optimizer = self._prepare_units(model, optimizer)
            if scheduler is not None:
                scheduler = AccumScheduler(scheduler, self.gradient_state)
            return model, optimizer, dataloader, scheduler
        model = self._prepare_model(model)
        self._fused = False
        if optimizer is not None:
            if hasattr(optimizer, "attach_flat"):
                use_reducer = self._reducer is not None and hasattr(optimizer, "attach_reducer")
                optimizer.attach_flat(self.flat, shard=self.shard if get_world_size() > 1 else None,
                                      allocate=not use_reducer)
                if use_reducer:
                    optimizer.attach_reducer(self._reducer)
                    self._fused = True
                    self._reducer.install_hooks(model)
            elif get_world_size() > 1:
                log.warning("fsdp: optimizer %s cannot shard its state; gradients are all-reduced and every "
                            "rank updates the full model", type(optimizer).__name__)
                self.shard = None
            optimizer = AccumOptimizer(optimizer, self.gradient_state, self.flat, self._after_optimizer_step)
        if scheduler is not None:
            scheduler = AccumScheduler(scheduler, self.gradient_state)
        return model, optimizer, dataloader, scheduler

    def _sync_gradients(self) -> None:
        if self.units is not None:
            self.units.finish_backward()
            return
        ws = get_world_size()
        if ws <= 1:
            return
        if self._reducer is not None:
            if not self._fused:
                self._reducer.allreduce_grads()
            return
        g = self.flat.grad
        if self.shard is None:
            dist.all_reduce(g)
            g.div_(ws)
            return
        off, n = self.shard
        mine = g[off:off + n]
        if dist.get_backend() == "gloo":  # gloo has no reduce_scatter_tensor
            dist.all_reduce(g)
        else:
            dist.reduce_scatter_tensor(mine, g[: n * ws])
        mine.div_(ws)

    def _after_optimizer_step(self) -> None:
        if self.units is not None:
            self.units.invalidate()
            return
        ws = get_world_size()
        if ws <= 1 or self.shard is None:
            return
        if self._reducer is not None:
            return  # fused: the kernel already published the updated slice; unfused: full update everywhere
        off, n = self.shard
        data = self.flat.data
        if dist.get_backend() == "gloo":
            pieces = [torch.empty(n, dtype=data.dtype, device=data.device) for _ in range(ws)]
            dist.all_gather(pieces, data[off:off + n].clone())
            for r, piece in enumerate(pieces):
                data[r * n:(r + 1) * n].copy_(piece)
        else:
            dist.all_gather_into_tensor(data[: n * ws], data[off:off + n].clone())

    def unwrap_model(self, model: nn.Module) -> Dict[str, torch.Tensor]:
        if self.units is not None:
            return self.units.full_state_dict()
        # parameters are kept whole between steps, so the local state dict is the full one
        return {k: v.detach().clone() for k, v in model.state_dict().items()}

    def grad_norm_sq_extra(self) -> Optional[torch.Tensor]:
        if self.units is not None:
            return self.units.grad_norm_sq() if get_world_size() > 1 else None
        if get_world_size() <= 1 or self.shard is None:
            return None
        off, n = self.shard
        sq = self.flat.grad[off:off + n].float().pow(2).sum()
        dist.all_reduce(sq)
        return sq


@ExecutorFactory.register("fsdp_block")
class BlockShardExecutor(FSDPExecutor):
    """``fsdp`` that insists on sharding the parameters block by block (raises where it cannot)."""

    default_shard_parameters = True


@ExecutorFactory.register("fsdp_zero1")
class ZeroOneExecutor(FSDPExecutor):
    """``fsdp`` with whole parameters and gradients resident: only the optimizer state and the update
    are sharded (works with every model and optimizer, adapters and CUDA-graph capture included)."""

    default_shard_parameters = False


def _hybrid_groups(tp_size: int):
    """Process groups of a ``dp x tp`` layout: tensor-parallel groups are runs of ``tp_size``
    consecutive ranks (same NVLink island), data-parallel groups take one rank of every run.
    Collective: every rank creates every group, in the same order."""
    ws, rank = get_world_size(), get_rank()
    if ws % tp_size:
        raise ValueError(f"world size {ws} is not a multiple of tp_size {tp_size}")
    tp_group = dp_group = None
    for start in range(0, ws, tp_size):
        g = dist.new_group(list(range(start, start + tp_size)))
        if start <= rank < start + tp_size:
            tp_group = g
    for offset in range(tp_size):
        g = dist.new_group(list(range(offset, ws, tp_size)))
        if rank % tp_size == offset:
            dp_group = g
    return tp_group, dp_group


@ExecutorFactory.register("tp")
class TPExecutor(BaseExecutor):
    """Tensor parallelism with sequence-sharded activations, optionally combined with data
    parallelism (``tp_size`` < world size: ``world / tp_size`` replicas of a ``tp_size``-way model).

    ``prepare`` rewrites the model into its tensor-parallel form (``khaosz_b200.parallel.tp_model``),
    points the optimizer at the sharded parameters, and makes every rank read the same batches
    (one data replica).  ``backward`` scales the local loss by ``1 / ws`` (each rank holds
    ``tokens / ws`` of the batch) and, on synchronisation steps, sums the gradients of the
    replicated parameters over the group.  ``unwrap_model`` returns the full state dict with
    the reference's parameter names.  The reference has no counterpart: its ``parallel_mode``
    choices are ``none/ddp/fsdp`` (``scripts/tools/train.py:171-176``).
    """

    def __init__(self, grad_accum_steps: int = 1, tp_size: Optional[int] = None, init_sync: bool = True,
                 fp8: bool = False, cuda_graph: bool = False, **_ignored):
        # fp8 covers the GEMMs that run locally (embedding-side LM head); the fused
        # collective GEMMs of the tensor-parallel layers are bf16
        super().__init__(grad_accum_steps, fp8, cuda_graph)
        self.tp_size = tp_size
        self.init_sync = init_sync
        self.tp_group = self.dp_group = None   # None: the tensor-parallel group is the whole world
        self.dp_size, self.dp_rank = 1, 0

    def _tp_ranks(self) -> int:
        return self.tp_size if self.tp_group is not None else get_world_size()

    def _prepare_model(self, model: nn.Module) -> nn.Module:
        from .tp_model import tensorize

        ws = get_world_size()
        if self.tp_size not in (None, ws) and ws > 1:
            self.tp_group, self.dp_group = _hybrid_groups(int(self.tp_size))
            self.dp_size, self.dp_rank = ws // self.tp_size, get_rank() // self.tp_size
        if self.init_sync:
            _broadcast_parameters(model, None)
        tp = tensorize(model, self.tp_group) if ws > 1 or dist.is_initialized() else model
        if self.flatten_on_cuda and _wants_flat(tp):
            self.flat = FlatParameters(tp, with_grad=True)
        self._model = tp
        return tp

    def prepare(self, model, optimizer=None, dataloader=None, scheduler=None):
        model = self._prepare_model(model)
        sampler = getattr(dataloader, "sampler", None)
        if hasattr(sampler, "set_replicas"):
            sampler.set_replicas(self.dp_size, self.dp_rank)   # the ranks of one model replica read the same data
        if optimizer is not None:
            if len(optimizer.param_groups) != 1:
                raise NotImplementedError("tp: optimizers with several parameter groups are not re-pointed")
            seen, params = set(), []
            for p in model.parameters():
                if p.requires_grad and id(p) not in seen:
                    seen.add(id(p))
                    params.append(p)
            optimizer.param_groups[0]["params"] = params
            optimizer.state.clear()
            if self.flat is not None and hasattr(optimizer, "attach_flat"):
                optimizer.attach_flat(self.flat)
            if hasattr(optimizer, "set_norm_fn") and hasattr(model, "grad_norm_sq"):
                optimizer.set_norm_fn(model.grad_norm_sq)
            optimizer = RankStateOptimizer(optimizer, self.gradient_state, self.flat, self._after_optimizer_step,
                                           group=self.tp_group, model=model)
        if scheduler is not None:
            scheduler = AccumScheduler(scheduler, self.gradient_state)
        return model, optimizer, dataloader, scheduler

    def _backward_only(self, loss: torch.Tensor) -> None:
        n = self._tp_ranks()
        (loss / n if n > 1 else loss).backward()

    def _sync_gradients(self) -> None:
        reduce = getattr(self._model, "reduce_replicated_grads", None)
        if reduce is not None:
            reduce()
        if self.dp_group is not None and self.dp_size > 1:   # average over the model replicas
            if self.flat is not None and self.flat.grad is not None:
                dist.all_reduce(self.flat.grad, group=self.dp_group)
                self.flat.grad.div_(self.dp_size)
            else:
                for p in self._model.parameters():
                    if p.grad is not None:
                        dist.all_reduce(p.grad, group=self.dp_group)
                        p.grad.div_(self.dp_size)

    def unwrap_model(self, model: nn.Module) -> Dict[str, torch.Tensor]:
        full = getattr(model, "full_state_dict", None)
        return full() if full is not None else model.state_dict()

    def grad_norm_sq_extra(self) -> Optional[torch.Tensor]:
        fn = getattr(self._model, "grad_norm_sq", None)
        return fn() if fn is not None and get_world_size() > 1 else None


@ExecutorFactory.register("fsdp_full")
class FullShardExecutor(TPExecutor):
    """Fully sharded data parallel: block weights exist as row shards, every forward / backward
    GEMM gathers its weight inside the kernel and reduce-scatters its weight gradient
    (``khaosz_b200.parallel.fsdp_model``).  Each rank trains on its own batches, owns the
    optimizer state of its shards and updates them without any further collective; the
    replicated embedding / norm gradients take one all-reduce per optimizer step.  This is the
    memory behaviour of the reference's ``ShardingStrategy.FULL_SHARD`` wrapper
    (``astrai/parallel/executor.py:223-272``); the ``fsdp`` executor keeps whole parameters
    resident and shards only gradients and optimizer state, which is faster while the model fits.
    """

    def _prepare_model(self, model: nn.Module) -> nn.Module:
        from .fsdp_model import full_shard

        if self.init_sync:
            _broadcast_parameters(model, None)
        fs = full_shard(model) if dist.is_initialized() else model
        if self.flatten_on_cuda and _wants_flat(fs):
            self.flat = FlatParameters(fs, with_grad=True)
        self._model = fs
        return fs

    def prepare(self, model, optimizer=None, dataloader=None, scheduler=None):
        sampler = getattr(dataloader, "sampler", None)
        replicas = (sampler.num_replicas, sampler.rank) if hasattr(sampler, "set_replicas") else None
        out = super().prepare(model, optimizer, dataloader, scheduler)
        if replicas is not None:
            sampler.set_replicas(*replicas)  # data parallel: every rank keeps its own slice of the data
        return out
