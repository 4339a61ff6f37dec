"""Symmetric-memory communication runtime for the executors.

``SymmetricBuffer`` allocates a buffer with ``torch.distributed._symmetric_memory`` so that
every rank of the group can address every peer's copy (and, on NVSwitch systems, a multicast
address that reaches all copies at once).  ``GradReducer`` re-homes an executor's flat
parameter and gradient buffers into such memory and runs the fused
reduce-scatter + clip + sharded AdamW + all-gather kernels of ``csrc/comm.cu`` once per
optimizer step; NCCL is only used for bootstrap and as the comparison path.

Environment: ``KHAOSZ_B200_NVLS=0`` forces plain peer loads/stores even where multicast is
available, and keeps torch's symmetric memory from creating or binding a multicast object at
all (``TORCH_SYMM_MEM_DISABLE_MULTICAST=1`` is set before the first rendezvous), so "NVLS off"
means that no rank's memory is ever bound to one (fault-tolerance tests require that).
"""

from __future__ import annotations

import ctypes
import os
from typing import Dict, List, Optional

import torch
import torch.distributed as dist

from ..ops import _lib
from ..ops._lib import check, lib, ptr, stream
from ..utils.flat_params import FlatParameters


def _ptr_array(values: List[int]):
    arr = (ctypes.c_void_p * len(values))(*values)
    return arr


class SymmetricBuffer:
    """A tensor whose peers' copies are addressable from this rank's kernels."""

    def __init__(self, numel: int, dtype: torch.dtype, device, group=None, zero: bool = True):
        if os.environ.get("KHAOSZ_B200_NVLS", "1") == "0":
            os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        import torch.distributed._symmetric_memory as symm

        self.group = group if group is not None else dist.group.WORLD
        self.tensor = symm.empty(numel, dtype=dtype, device=device)
        if zero:
            self.tensor.zero_()
        self.handle = symm.rendezvous(self.tensor, self.group)
        self.rank, self.world_size = self.handle.rank, self.handle.world_size
        self.peer_ptrs = [int(p) for p in self.handle.buffer_ptrs]
        self._ptr_array = _ptr_array(self.peer_ptrs)
        mc = 0
        try:
            if os.environ.get("KHAOSZ_B200_NVLS", "1") != "0" and self.handle.has_multicast_support(
                    self.tensor.device.type, self.tensor.device.index):
                mc = int(self.handle.multicast_ptr or 0)
        except Exception:
            mc = 0
        self.multicast_ptr = mc

    @property
    def ptrs(self):
        return self._ptr_array


class PeerControl:
    """Epoch counters for the in-kernel barriers plus the slots for exchanged scalars."""

    def __init__(self, device, group=None):
        slots = lib().kb_comm_slots()
        self.flags = SymmetricBuffer(slots * 8, torch.int32, device, group)
        self.norms = SymmetricBuffer(64, torch.float32, device, group)
        self.epoch = 4
        torch.cuda.synchronize(device)
        dist.barrier(group=self.flags.group)  # every rank's zero-fill has landed before first use

    def next_epoch(self, n: int = 4) -> int:
        e = self.epoch
        self.epoch += n
        return e

    def barrier(self, budget_ms: int = 0, slot: Optional[int] = None) -> None:
        f = self.flags
        slot = lib().kb_comm_slots() - 1 if slot is None else slot
        check(lib().kb_peer_barrier(f.ptrs, f.rank, f.world_size, slot, self.next_epoch(), budget_ms, stream()),
              "peer_barrier")


def allreduce_(buf: SymmetricBuffer, ctrl: PeerControl, scale: float = 1.0, use_multicast: bool = True) -> torch.Tensor:
    """In-place sum (times ``scale``) over the ranks of a symmetric bf16 buffer."""
    assert buf.tensor.dtype == torch.bfloat16 and buf.tensor.numel() % 8 == 0
    mc = buf.multicast_ptr if use_multicast else 0
    check(lib().kb_allreduce_bf16(buf.ptrs, ctrl.flags.ptrs, ctypes.c_void_p(mc) if mc else None, buf.rank,
                                  buf.world_size, buf.tensor.numel(), float(scale), ctrl.next_epoch(), stream()),
          "allreduce_bf16")
    return buf.tensor


def _mc(buf: SymmetricBuffer, use_multicast: bool):
    return ctypes.c_void_p(buf.multicast_ptr) if (use_multicast and buf.multicast_ptr) else None


def reduce_scatter(buf: SymmetricBuffer, ctrl: PeerControl, out: Optional[torch.Tensor] = None, scale: float = 1.0,
                   use_multicast: bool = True) -> torch.Tensor:
    """``out = scale * sum over ranks of piece[rank]`` of a symmetric bf16 buffer (``numel`` a multiple of
    ``8 * world_size``); ``out`` defaults to a fresh local tensor of ``numel / world_size`` elements."""
    n = buf.tensor.numel()
    assert buf.tensor.dtype == torch.bfloat16 and n % (8 * buf.world_size) == 0
    if out is None:
        out = torch.empty(n // buf.world_size, dtype=torch.bfloat16, device=buf.tensor.device)
    check(lib().kb_reducescatter_bf16(buf.ptrs, ctrl.flags.ptrs, _mc(buf, use_multicast), buf.rank, buf.world_size, n,
                                      float(scale), ptr(out), ctrl.next_epoch(2), stream()), "reducescatter_bf16")
    return out


def all_gather_(buf: SymmetricBuffer, ctrl: PeerControl, use_multicast: bool = True) -> torch.Tensor:
    """Every rank's piece ``[rank * n / ws, (rank + 1) * n / ws)`` of the symmetric buffer lands in all copies."""
    n = buf.tensor.numel()
    assert buf.tensor.dtype == torch.bfloat16 and n % (8 * buf.world_size) == 0
    check(lib().kb_allgather_bf16(buf.ptrs, ctrl.flags.ptrs, _mc(buf, use_multicast), buf.rank, buf.world_size, n,
                                  ctrl.next_epoch(2), stream()), "allgather_bf16")
    return buf.tensor


def broadcast_(buf: SymmetricBuffer, ctrl: PeerControl, root: int = 0, numel: Optional[int] = None,
               use_multicast: bool = True) -> torch.Tensor:
    """The first ``numel`` elements (default: all; a multiple of 8) of ``root``'s copy land in every copy."""
    n = buf.tensor.numel() if numel is None else numel
    assert buf.tensor.dtype == torch.bfloat16 and n % 8 == 0
    check(lib().kb_broadcast_bf16(buf.ptrs, ctrl.flags.ptrs, _mc(buf, use_multicast), root, buf.rank, buf.world_size, n,
                                  ctrl.next_epoch(4), stream()), "broadcast_bf16")
    return buf.tensor


class GradReducer:
    """Owns the symmetric homes of an executor's flat buffers and the fused optimizer step.

    The flat gradient buffer is cut into buckets of about ``bucket_cap_mb`` (the reference's
    ``DDPExecutor(bucket_cap_mb=25)``, ``astrai/parallel/executor.py:146-198``); rank ``r`` owns
    sub-slice ``r`` of every bucket.  With ``overlap`` (executor keyword ``overlap_grad_reduce=True`` or
    ``KHAOSZ_B200_DDP_OVERLAP=1``) the buckets of the micro-batch that ends an accumulation window
    are reduced *while the backward pass is still running*: as soon as every parameter of a bucket has
    received its last gradient contribution (and all later buckets have been handed over), the
    bucket's reduce-scatter kernel is launched on a side stream behind an event, with a small grid
    that shares the SMs with the backward kernels.  What is left when the backward pass returns is
    flushed, then one exchange of the squared-norm partials, the clip factor, the sharded AdamW and
    the parameter all-gather run as before.  Buckets are always handed over in the same (descending)
    order on every rank, whatever the timing, because the kernels of the ranks pair up by call order.
    """

    fuses_optimizer = True
    gathers_params = True
    BUCKET_GRID = 48        # CTAs of a bucket reduction (the same on every rank: per-CTA barriers pair up)
    BUCKET_THREADS = 256    # light enough to be co-resident with a persistent GEMM CTA

    def __init__(self, flat: FlatParameters, mode: str, group=None, bucket_cap_mb: Optional[float] = None,
                 overlap: Optional[bool] = None):
        dev = flat.data.device
        self.flat, self.mode = flat, mode
        ws = dist.get_world_size(group)
        if flat.numel % (8 * ws):
            raise ValueError("flat buffer length must be a multiple of 8 * world_size")
        self.params = SymmetricBuffer(flat.numel, flat.data.dtype, dev, group, zero=False)
        self.grads = SymmetricBuffer(flat.numel, flat.data.dtype, dev, group, zero=True)
        self.params.tensor.copy_(flat.data)
        flat.rebind(self.params.tensor, self.grads.tensor)
        self.ctrl = PeerControl(dev, group)
        self.rank, self.ws = self.params.rank, ws
        self.slice_n = flat.numel // ws
        unit = 8 * ws
        if overlap is None:
            # off unless asked for: in every configuration measured so far (8 and 1 micro-batches per step,
            # 2 and 8 GPUs) the bucket kernels that share the SMs with the backward pass cost more than
            # the few milliseconds of reduction they hide
            overlap = os.environ.get("KHAOSZ_B200_DDP_OVERLAP", "0") == "1"
        bucket_n = flat.numel
        if overlap and bucket_cap_mb and bucket_cap_mb > 0 and _lib.has("kb_reduce_bucket"):
            bucket_n = max(unit, int(bucket_cap_mb * 2 ** 20) // flat.data.element_size() // unit * unit)
        self.bucket_n = min(bucket_n, flat.numel)
        self.n_buckets = -(-flat.numel // self.bucket_n)
        self.overlap = bool(overlap) and self.n_buckets > 1
        self.slice_off = self.rank * self.slice_n if self.n_buckets == 1 else None
        self._m = torch.zeros(self.slice_n, dtype=torch.float32, device=dev)
        self._v = torch.zeros(self.slice_n, dtype=torch.float32, device=dev)
        self._scratch = torch.zeros(2, dtype=torch.float32, device=dev)
        self._lr_dev = torch.zeros(2, dtype=torch.float32, device=dev)
        self.use_multicast = bool(self.params.multicast_ptr and self.grads.multicast_ptr)
        # bucket bookkeeping for the overlapped hand-over
        self._comm_stream = torch.cuda.Stream(device=dev) if self.overlap else None
        self._bucket_params: List[List[int]] = [[] for _ in range(self.n_buckets)]   # indices into flat.params
        self._param_buckets: Dict[int, List[int]] = {}
        for i, (p, off) in enumerate(zip(flat.params, flat.offsets)):
            if not p.requires_grad or p.numel() == 0:
                continue
            bs = list(range(off // self.bucket_n, (off + p.numel() - 1) // self.bucket_n + 1))
            self._param_buckets[id(p)] = bs
            for b in bs:
                self._bucket_params[b].append(i)
        self._armed = False
        self._remaining: List[int] = []
        self._next_bucket = -1
        self._late: set = set()
        self._used_side_stream = False
        self.buckets_overlapped = 0   # buckets handed over before the backward pass returned (last window)

    @classmethod
    def create(cls, flat: FlatParameters, mode: str = "allreduce", group=None, bucket_cap_mb: Optional[float] = None,
               overlap: Optional[bool] = None) -> Optional["GradReducer"]:
        if not (flat.data.is_cuda and flat.data.dtype == torch.bfloat16 and _lib.has("kb_reduce_adamw")):
            return None
        ws = dist.get_world_size(group)
        if ws > 8 or flat.numel % (8 * ws):
            return None
        return cls(flat, mode, group, bucket_cap_mb, overlap)

    # -- layout ---------------------------------------------------------------------------------
    def bucket_range(self, b: int):
        lo = b * self.bucket_n
        return lo, min(self.bucket_n, self.flat.numel - lo)

    def owned_ranges(self, rank: Optional[int] = None):
        """``(global_offset, local_offset, n)`` of the pieces of the flat vector whose optimizer state
        lives on ``rank`` (this rank by default), in the order the moments are stored."""
        rank = self.rank if rank is None else rank
        out, local = [], 0
        for b in range(self.n_buckets):
            lo, n = self.bucket_range(b)
            piece = n // self.ws
            out.append((lo + rank * piece, local, piece))
            local += piece
        return out

    # -- hand-over of finished buckets --------------------------------------------------------------
    def install_hooks(self, model) -> None:
        """Tell this reducer when a parameter's gradient is final for the micro-batch.  Linear weights
        report through the layer functions (``ops.functional.set_grad_ready_hook``); every other
        parameter through autograd's post-accumulation hook, counted against the forward calls of its
        module.  A parameter that is fed both ways (a tied embedding / output weight) counts as late
        and goes with the final flush."""
        if not self.overlap:
            return
        from ..models.components.layers import Linear
        from ..ops import functional

        if any(hasattr(m, "n_routed_experts") for m in model.modules()):
            # data-dependent expert routing: which parameters receive a gradient differs from rank to
            # rank, and with it the moment a bucket is complete; the ranks' launches must pair up, so
            # such models reduce everything in one launch after the backward pass
            self.overlap = False
            return

        linear_w = {id(m.weight) for m in model.modules() if isinstance(m, Linear)}
        for module in model.modules():
            direct = [p for p in module.parameters(recurse=False) if p.requires_grad and id(p) in self._param_buckets]
            if not direct:
                continue
            if isinstance(module, Linear):
                continue
            for p in direct:
                if id(p) in linear_w:
                    self._late.add(id(p))
            others = [p for p in direct if id(p) not in linear_w]
            if not others:
                continue

            def count(mod, args, _ps=others):
                if self._armed and torch.is_grad_enabled():
                    for p in _ps:
                        p._kb_uses = getattr(p, "_kb_uses", 0) + 1

            module.register_forward_pre_hook(count)
            for p in others:
                def done(param):
                    if self._armed:
                        param._kb_done = getattr(param, "_kb_done", 0) + 1
                        if param._kb_done >= getattr(param, "_kb_uses", 0):
                            self.notify(param)

                p.register_post_accumulate_grad_hook(done)
        functional.set_grad_ready_hook(self.notify)

    def begin_window(self, final: bool) -> None:
        """Called before the forward pass of every micro-batch; ``final``: this one ends the window."""
        if not self.overlap:
            return
        self._armed = bool(final)
        if not final:
            return
        for p in self.flat.params:
            p._kb_uses = 0
            p._kb_done = 0
        self._remaining = [sum(1 for i in idx if id(self.flat.params[i]) not in self._late) +
                           (10 ** 9 if any(id(self.flat.params[i]) in self._late for i in idx) else 0)
                           for idx in self._bucket_params]
        self._next_bucket = self.n_buckets - 1
        self._used_side_stream = False
        self.buckets_overlapped = 0
        self._scratch.zero_()

    def notify(self, p) -> None:
        if not self._armed:
            return
        for b in self._param_buckets.get(id(p), ()):
            self._remaining[b] -= 1
        self._hand_over(side=True)

    def _launch_range(self, b_lo: int, b_hi: int, side: bool) -> None:
        """Reduce-scatter of the buckets ``b_lo .. b_hi``: one finished bucket on the side stream behind
        an event (small grid of light CTAs), or whatever is left in one launch with the full grid."""
        mc_g = ctypes.c_void_p(self.grads.multicast_ptr) if self.use_multicast else None
        main = torch.cuda.current_stream()
        if side and self._comm_stream is not None:
            ev = torch.cuda.Event()
            ev.record(main)
            self._comm_stream.wait_event(ev)
            st = ctypes.c_void_p(self._comm_stream.cuda_stream)
            self._used_side_stream = True
            self.buckets_overlapped += b_hi - b_lo + 1
            grid, threads = self.BUCKET_GRID, self.BUCKET_THREADS
        else:
            if self._used_side_stream:      # keep the buckets in one order on the device as well
                ev = torch.cuda.Event()
                ev.record(self._comm_stream)
                main.wait_event(ev)
            st = stream()
            grid, threads = lib().kb_comm_slots() - 8, 512
        check(lib().kb_reduce_bucket(self.grads.ptrs, self.ctrl.flags.ptrs, mc_g, self.rank, self.ws, self.bucket_n,
                                     self.flat.numel, b_lo, b_hi, ptr(self._scratch), self.ctrl.next_epoch(1), grid,
                                     threads, st), "reduce_bucket")

    def _hand_over(self, side: bool, flush: bool = False) -> None:
        if flush:
            if self._next_bucket >= 0:
                self._launch_range(0, self._next_bucket, side=False)
                self._next_bucket = -1
            return
        while self._next_bucket >= 0 and self._remaining[self._next_bucket] <= 0:
            self._launch_range(self._next_bucket, self._next_bucket, side)
            self._next_bucket -= 1

    def reduce(self) -> None:
        """Gradient reduction is part of :meth:`fused_step`; nothing to do at backward time."""

    def allreduce_grads(self) -> None:
        """Stand-alone mean all-reduce of the gradient buffer (for optimizers that cannot fuse)."""
        self._armed = False
        allreduce_(self.grads, self.ctrl, 1.0 / self.ws, self.use_multicast)

    def fused_step(self, opt, lr, beta1, beta2, eps, wd, clip, step) -> None:
        _lib.set_device_floats(self._lr_dev, lr, step)   # launch arguments: no staging buffer to overwrite
        mc_p = ctypes.c_void_p(self.params.multicast_ptr) if self.use_multicast else None
        if self.n_buckets == 1:
            mc_g = ctypes.c_void_p(self.grads.multicast_ptr) if self.use_multicast else None
            check(lib().kb_reduce_adamw(self.grads.ptrs, self.params.ptrs, self.ctrl.flags.ptrs, self.ctrl.norms.ptrs,
                                        mc_g, mc_p, self.rank, self.ws, self.slice_off, self.slice_n, ptr(self._m),
                                        ptr(self._v), ptr(self._lr_dev), beta1, beta2, eps, wd, float(clip or 0.0),
                                        ptr(self._scratch), self.ctrl.next_epoch(), stream()), "reduce_adamw")
            _lib.add_launches(2)
        else:
            if not self._armed:             # nobody announced the window (direct use): everything now
                self._scratch.zero_()
                self._next_bucket = self.n_buckets - 1
                self._used_side_stream = False
                self.buckets_overlapped = 0
            self._hand_over(side=False, flush=True)
            self._armed = False
            if self._used_side_stream:
                ev = torch.cuda.Event()
                ev.record(self._comm_stream)
                torch.cuda.current_stream().wait_event(ev)
            check(lib().kb_adamw_buckets(self.grads.ptrs, self.params.ptrs, self.ctrl.flags.ptrs, self.ctrl.norms.ptrs,
                                         mc_p, self.rank, self.ws, self.bucket_n, self.flat.numel, ptr(self._m),
                                         ptr(self._v), ptr(self._lr_dev), beta1, beta2, eps, wd, float(clip or 0.0),
                                         ptr(self._scratch), self.ctrl.next_epoch(2), stream()), "adamw_buckets")
            _lib.add_launches(1)
        opt.last_grad_norm = self._scratch[1:2].sqrt()

    # optimizer-state plumbing used by FusedAdamW.state_dict / load_state_dict
    def moments(self):
        shard = (self.slice_off, self.slice_n) if self.n_buckets == 1 else (0, self.slice_n)
        return self._m, self._v, shard
