"""Block-granular full sharding of a dense model's storage (ZeRO-3 behaviour).

The model keeps its modules, names and kernels; what changes is where its parameters live:

* every decoder block is one *unit*: its parameters are laid out in one flat vector of ``U``
  elements and rank ``r`` stores only elements ``[r * U / ws, (r + 1) * U / ws)`` of it, next to
  the gradient and the AdamW moments of that piece;
* two *weight images* and two *gradient images* of ``U`` elements exist per rank (the gradient
  images in symmetric memory on CUDA).  Block ``i`` computes out of image ``i % 2``: its parameters are permanent
  views of that image, so q/k/v and gate/up stay adjacent and every GEMM, fused epilogue and
  saved-for-backward view of the dense model works unchanged;
* before a block runs (forward and again backward) its unit is gathered into its image on a side
  stream: the rank's copy engine pulls every rank's piece over NVLink out of the symmetric memory
  the pieces live in.  The pieces only change in the optimizer step, which is fenced by a barrier
  on each side, so a gather needs neither a handshake with the peers nor an SM.  While block ``i``
  computes, block ``i + 1`` (forward) or ``i - 1`` (backward) is gathered into the other image;
* when a block's backward has finished, its gradient image is reduce-scattered by a kernel on the
  side stream (peer loads, or one ``multimem.ld_reduce`` through the switch), scaled by ``1 / ws``
  and added to the owned gradient piece; the same kernel clears the image, which is reused two
  blocks later.  Gathers and reductions have a stream each, so that a gather never queues behind a
  reduction;
* parameters outside the blocks (embedding, final norm, an untied output layer) stay replicated;
  their gradients take one all-reduce per optimizer step.

Per rank this holds ``1 / ws`` of the block weights, gradients and moments plus four images,
which is the memory behaviour of the reference's ``ShardingStrategy.FULL_SHARD`` wrapper
(``astrai/parallel/executor.py:223-272``: parameters gathered for each forward and backward,
gradients reduce-scattered).  Without CUDA (tests, gloo) the same schedule runs on plain tensors
with ``torch.distributed`` collectives on the calling thread.
"""

from __future__ import annotations

import ctypes
import os
from typing import Dict, List, Optional, Tuple

import torch
import torch.distributed as dist
import torch.nn as nn

ALIGN = 8     # elements: 16 bytes of bf16 (TMA and 128-bit accesses)


def _unique(params) -> List[nn.Parameter]:
    seen, out = set(), []
    for p in params:
        if id(p) not in seen:
            seen.add(id(p))
            out.append(p)
    return out


class _Unit:
    """Layout of one block's parameters inside its flat vector."""

    def __init__(self, params: List[nn.Parameter], ws: int):
        self.params = params
        self.offsets: List[int] = []
        off = 0
        for p in params:
            off = (off + ALIGN - 1) // ALIGN * ALIGN
            self.offsets.append(off)
            off += p.numel()
        pad = ALIGN * ws
        self.numel = (off + pad - 1) // pad * pad     # U
        self.per = self.numel // ws                   # owned piece
        self.base = 0          # offset of this unit in the dense (unsharded) coordinate system
        self.local = 0         # offset of the owned piece in the local shard vectors


class ShardedFlat:
    """What the optimizer and the executor see instead of a ``FlatParameters``: ``data`` / ``grad`` are
    the rank's local vectors (owned block pieces, then the replicated parameters); ``params`` /
    ``offsets`` / ``numel`` describe the dense layout (all units whole, then the replicated
    parameters), which is the coordinate system of checkpoints."""

    def __init__(self, params, offsets, numel, data, grad):
        self.params, self.offsets, self.numel = params, offsets, numel
        self.data, self.grad = data, grad

    def zero_grad(self) -> None:
        self.grad.zero_()


class _Enter(torch.autograd.Function):
    """Identity at a block's input: forward makes the block's weights resident, backward (the last
    node of the block's backward pass) hands its gradient image to the reduce-scatter."""

    @staticmethod
    def forward(ctx, x, units, i):
        ctx.units, ctx.i = units, i
        units._enter(i, forward=True)
        return x.view_as(x)

    @staticmethod
    def backward(ctx, g):
        ctx.units._reduce(ctx.i)
        return g, None, None


class _Exit(torch.autograd.Function):
    """Identity at a block's output: its backward is the first node of the block's backward pass and
    makes the weights resident again and the gradient image ready."""

    @staticmethod
    def forward(ctx, y, units, i):
        ctx.units, ctx.i = units, i
        return y.view_as(y)

    @staticmethod
    def backward(ctx, g):
        ctx.units._enter(ctx.i, forward=False)
        return g, None, None


class ShardedUnits:
    def __init__(self, model: nn.Module, group=None, prefetch: bool = True, frozen: bool = False):
        """``frozen``: a model that is only evaluated (the frozen copy of DPO / GRPO): no parameter requires a
        gradient, and neither gradient vectors nor gradient images exist."""
        if not isinstance(getattr(model, "layers", None), (nn.ModuleList, list, tuple)) or len(model.layers) == 0:
            raise NotImplementedError(f"block-granular sharding needs a model with a `layers` list, not {type(model).__name__}")
        self.model, self.group, self.prefetch, self.frozen = model, group, prefetch, frozen
        on = dist.is_available() and dist.is_initialized()
        self.ws = dist.get_world_size(group) if on else 1
        self.rank = dist.get_rank(group) if on else 0
        all_params = _unique(model.parameters())
        if frozen and any(p.requires_grad for p in all_params):
            raise ValueError("a frozen sharded copy must not have trainable parameters")
        if not frozen and not all(p.requires_grad for p in all_params):
            raise NotImplementedError("block-granular sharding trains every parameter (no frozen weights / adapters)")
        dtype, dev = all_params[0].dtype, all_params[0].device
        if any(p.dtype != dtype or p.device != dev for p in all_params):
            raise ValueError("block-granular sharding needs one dtype and one device for all parameters")
        self.dtype, self.device = dtype, dev
        self.cuda = dev.type == "cuda"

        # ---- layout ---------------------------------------------------------------------------
        self.units: List[_Unit] = []
        owner: Dict[int, int] = {}
        for i, block in enumerate(model.layers):
            ps = _unique(block.parameters())
            for p in ps:
                if id(p) in owner:
                    raise NotImplementedError("a parameter shared between blocks cannot be sharded by block")
                owner[id(p)] = i
            self.units.append(_Unit(ps, self.ws))
        self.rest = [p for p in all_params if id(p) not in owner]
        base = local = 0
        for u in self.units:
            u.base, u.local = base, local
            base += u.numel
            local += u.per
        self.rest_base, self.rest_local = base, local
        self.rest_offsets: List[int] = []
        off = 0
        for p in self.rest:
            off = (off + ALIGN - 1) // ALIGN * ALIGN
            self.rest_offsets.append(off)
            off += p.numel()
        self.rest_numel = (off + ALIGN - 1) // ALIGN * ALIGN
        self.dense_numel = self.rest_base + self.rest_numel
        self.local_numel = self.rest_local + self.rest_numel
        self.image_numel = max(u.numel for u in self.units)

        # ---- storage --------------------------------------------------------------------------
        self._sym = self.cuda and self.ws > 1
        if self._sym:
            from ..ops import _lib
            from .comm import PeerControl, SymmetricBuffer

            if dtype != torch.bfloat16 or not _lib.has("kb_unit_reduce_bf16"):
                raise RuntimeError("block-granular sharding on CUDA needs bf16 parameters and the collective kernels")
            if self.ws > 8:
                raise NotImplementedError("the collective kernels address at most 8 ranks")
            # the owned pieces live in symmetric memory: peers' copy engines read them when they gather a unit
            self._dbuf = SymmetricBuffer(self.local_numel, dtype, dev, group)
            self.data = self._dbuf.tensor
            self._gbuf = [] if frozen else [SymmetricBuffer(self.image_numel, dtype, dev, group) for _ in range(2)]
            self.g_image = [b.tensor for b in self._gbuf]
            self._ctrl = None if frozen else PeerControl(dev, group)   # its epochs order the side stream's reductions
            self._sync = PeerControl(dev, group)       # barriers on the main stream around the optimizer step
            # two side streams: a gather must never queue behind a reduction (the block after next waits for
            # the gather, nothing waits for the reduction before the image is reused)
            self._side = torch.cuda.Stream(device=dev)
            self._copy = torch.cuda.Stream(device=dev)
            # CTAs x threads of the reduce kernel (the same on every rank; 0: one CTA per SM).  Measured on the
            # 1B model: a reduction spread over all SMs and finished quickly costs less than a small grid
            # that lingers beside the compute kernels (12 / 32 / 96 / 148 CTAs: 674 / 628 / 617 / 608 ms per step)
            self.grid = int(os.environ.get("KHAOSZ_B200_SHARD_GRID", "0"))
            self.threads = int(os.environ.get("KHAOSZ_B200_SHARD_THREADS", "256"))
        else:
            self.data = torch.zeros(self.local_numel, dtype=dtype, device=dev)
            self.g_image = [] if frozen else [torch.zeros(self.image_numel, dtype=dtype, device=dev) for _ in range(2)]
            self._side = self._copy = None
        self.grad = None if frozen else torch.zeros(self.local_numel, dtype=dtype, device=dev)
        self.w_image = [torch.zeros(self.image_numel, dtype=dtype, device=dev) for _ in range(2)]
        self._content = [-1, -1]          # which unit each weight image holds
        self._ready = [None, None]        # event: the image's last gather has landed
        self._reduced = [None, None]      # event: the gradient image's last reduce-scatter is done
        self.gathers = self.reductions = 0

        # ---- move the parameters ------------------------------------------------------------------
        with torch.no_grad():
            for i, u in enumerate(self.units):
                lo = self.rank * u.per
                full = torch.zeros(u.numel, dtype=dtype, device=dev)
                for p, o in zip(u.params, u.offsets):
                    full[o:o + p.numel()].copy_(p.data.reshape(-1))
                self.data[u.local:u.local + u.per].copy_(full[lo:lo + u.per])
                w = self.w_image[i % 2]
                for p, o in zip(u.params, u.offsets):
                    p.data = w[o:o + p.numel()].view(p.shape)
                    p.grad = None
                    if not frozen:
                        p.main_grad = self.g_image[i % 2][o:o + p.numel()].view(p.shape)
                del full
            for p, o in zip(self.rest, self.rest_offsets):
                lo = self.rest_local + o
                view = self.data[lo:lo + p.numel()].view(p.shape)
                view.copy_(p.data)
                p.data = view
                if not frozen:
                    p.main_grad = self.grad[lo:lo + p.numel()].view(p.shape)
                    p.grad = p.main_grad
        params, offsets = [], []
        where = {id(p): u.base + o for u in self.units for p, o in zip(u.params, u.offsets)}
        where.update({id(p): self.rest_base + o for p, o in zip(self.rest, self.rest_offsets)})
        for p in all_params:      # optimizer order = model.parameters() order, as in a dense run
            params.append(p)
            offsets.append(where[id(p)])
        self.flat = ShardedFlat(params, offsets, self.dense_numel, self.data, self.grad)

        if self._sym:
            self._sync.barrier()      # every rank's pieces are in place before anyone gathers
        for i, block in enumerate(model.layers):
            block.register_forward_pre_hook(self._pre_hook(i), with_kwargs=True)
            block.register_forward_hook(self._post_hook(i))

    # ---- hooks ------------------------------------------------------------------------------------
    def _pre_hook(self, i: int):
        def hook(module, args, kwargs):
            if not args:
                raise RuntimeError("a sharded block takes its hidden states as the first positional argument")
            x = args[0]
            if torch.is_grad_enabled() and not x.requires_grad and not self.frozen:
                x = x.detach().requires_grad_()     # the block's backward must reach its input node
            return (_Enter.apply(x, self, i),) + tuple(args[1:]), kwargs
        return hook

    def _post_hook(self, i: int):
        def hook(module, args, output):
            if torch.is_grad_enabled() and isinstance(output, torch.Tensor) and output.requires_grad:
                return _Exit.apply(output, self, i)
            return output
        return hook

    # ---- schedule -----------------------------------------------------------------------------------
    def _gather(self, i: int) -> None:
        """Unit ``i`` into weight image ``i % 2`` (asynchronously on the copy stream on CUDA)."""
        u, s = self.units[i], i % 2
        mine = self.data[u.local:u.local + u.per]
        self.gathers += 1
        from ..ops.functional import bump_weight_generation, fp8_linear_enabled

        if fp8_linear_enabled():
            bump_weight_generation()    # fp8 weight images are cached by address, and blocks share the images
        if self._sym:
            from ..ops._lib import check, lib

            main = torch.cuda.current_stream()
            ev = torch.cuda.Event()
            ev.record(main)                 # everything that read the image's old content is queued before this
            self._copy.wait_event(ev)
            # pull: this rank's copy engine reads every rank's piece (its own included) into its own image.  The
            # pieces only change in the optimizer step, which is fenced by barriers on both sides, so a gather
            # needs no handshake with the peers and no SM
            w, side, nbytes = self.w_image[s], ctypes.c_void_p(self._copy.cuda_stream), u.per * mine.element_size()
            for k in range(self.ws):
                r = (self.rank + k) % self.ws
                check(lib().kb_copy_async(ctypes.c_void_p(w.data_ptr() + r * nbytes),
                                          ctypes.c_void_p(self._dbuf.peer_ptrs[r] + u.local * mine.element_size()),
                                          nbytes, side), "copy_async")
            done = torch.cuda.Event()
            done.record(self._copy)
            self._ready[s] = done
        else:
            w = self.w_image[s]
            with torch.no_grad():
                if self.ws > 1:
                    dist.all_gather([w[r * u.per:(r + 1) * u.per] for r in range(self.ws)], mine.clone(),
                                    group=self.group)
                else:
                    w[:u.per].copy_(mine)
        self._content[s] = i

    def _enter(self, i: int, forward: bool) -> None:
        s = i % 2
        if self._content[s] != i:
            self._gather(i)
        if self._sym and self._ready[s] is not None:
            torch.cuda.current_stream().wait_event(self._ready[s])
        if not forward and not self.frozen:
            u = self.units[i]
            if self._sym and self._reduced[s] is not None:
                torch.cuda.current_stream().wait_event(self._reduced[s])   # the image's previous user has been reduced
            if not self._sym:      # on CUDA the reduce kernel leaves the image cleared
                with torch.no_grad():
                    self.g_image[s][:u.numel].zero_()
            for p in u.params:
                if p.grad is None:
                    p.grad = p.main_grad
        if self.prefetch and self.ws > 1:
            j = i + 1 if forward else i - 1
            # the other image's last user (block i - 1 forward, block i + 1 backward) is queued already
            if 0 <= j < len(self.units) and self._content[j % 2] != j:
                self._gather(j)

    def _reduce(self, i: int) -> None:
        """Block ``i``'s backward is complete: mean of its gradient image over the ranks, added to the
        owned gradient piece."""
        if self.frozen:         # gradients flow through a frozen copy, none is kept
            return
        u, s = self.units[i], i % 2
        mine = self.grad[u.local:u.local + u.per]
        lo = self.rank * u.per
        self.reductions += 1
        if self._sym:
            from ..ops._lib import check, lib, ptr

            ev = torch.cuda.Event()
            ev.record(torch.cuda.current_stream())
            self._side.wait_event(ev)
            buf = self._gbuf[s]
            mc = ctypes.c_void_p(buf.multicast_ptr) if buf.multicast_ptr else None
            # the kernel adds the mean to the owned piece and, once every rank has read, clears this rank's image
            check(lib().kb_unit_reduce_bf16(buf.ptrs, self._ctrl.flags.ptrs, mc, self.rank, self.ws, u.numel,
                                            1.0 / self.ws, ptr(mine), 1, self._ctrl.next_epoch(2), self.grid, self.threads,
                                            ctypes.c_void_p(self._side.cuda_stream)), "unit_reduce")
            done = torch.cuda.Event()
            done.record(self._side)
            self._reduced[s] = done
        else:
            g = self.g_image[s]
            with torch.no_grad():
                if self.ws > 1:
                    dist.all_reduce(g[:u.numel], group=self.group)
                mine.add_(g[lo:lo + u.per] / self.ws)
        # the image now belongs to the block after next: outside its own backward pass a block's parameters
        # carry no ``.grad`` (per-parameter gradient statistics then skip them instead of reading an image)
        for p in u.params:
            p.grad = None

    def finish_backward(self) -> None:
        """Called once per optimizer step before the update: the side stream's reductions have to be
        complete, and the replicated parameters' gradients are averaged."""
        if self.frozen:
            return
        if self._sym:
            for ev in self._reduced:
                if ev is not None:
                    torch.cuda.current_stream().wait_event(ev)
        if self.ws > 1 and self.rest_numel:
            g = self.grad[self.rest_local:]
            dist.all_reduce(g, group=self.group)
            g.div_(self.ws)
        if self._sym:
            # no rank changes its pieces while a peer may still be gathering them: every rank's main stream has
            # waited for its last gather when it arrives here
            self._sync.barrier()

    def invalidate(self) -> None:
        """The owned pieces changed (optimizer step, loaded weights): the images are stale, and no rank
        gathers before every rank's pieces are final."""
        self._content = [-1, -1]
        if self._sym:
            self._sync.barrier()

    # ---- norms, state ---------------------------------------------------------------------------------
    @torch.no_grad()
    def grad_norm_sq(self) -> torch.Tensor:
        """Global squared gradient norm (call after :meth:`finish_backward`)."""
        sharded = self._sumsq(self.grad[:self.rest_local])
        if self.ws > 1:
            dist.all_reduce(sharded, group=self.group)
        return sharded + self._sumsq(self.grad[self.rest_local:])

    @staticmethod
    def _sumsq(t: torch.Tensor) -> torch.Tensor:
        if t.is_cuda and t.dtype == torch.bfloat16 and t.numel():
            from ..ops import _lib

            if _lib.has("kb_sumsq_bf16"):
                out = torch.zeros(1, dtype=torch.float32, device=t.device)
                _lib.check(_lib.lib().kb_sumsq_bf16(_lib.ptr(t), t.numel(), _lib.ptr(out), _lib.stream()), "sumsq")
                return out
        return t.float().pow(2).sum().reshape(1)

    def owned_ranges(self, rank: Optional[int] = None) -> List[Tuple[int, int, int]]:
        """``(dense offset, local offset, n)`` of what ``rank`` (default: this rank) stores."""
        r = self.rank if rank is None else rank
        out = [(u.base + r * u.per, u.local, u.per) for u in self.units]
        if self.rest_numel:
            out.append((self.rest_base, self.rest_local, self.rest_numel))
        return out

    @torch.no_grad()
    def _whole_unit(self, i: int, local_vec: torch.Tensor) -> torch.Tensor:
        u = self.units[i]
        mine = local_vec[u.local:u.local + u.per].contiguous()
        if self.ws == 1:
            return mine.clone()
        pieces = [torch.empty_like(mine) for _ in range(self.ws)]
        dist.all_gather(pieces, mine, group=self.group)
        return torch.cat(pieces)

    @torch.no_grad()
    def full_state_dict(self) -> Dict[str, torch.Tensor]:
        """The unsharded state dict with the dense model's names, identical on every rank (collective)."""
        values: Dict[int, torch.Tensor] = {}
        for i, u in enumerate(self.units):
            full = self._whole_unit(i, self.data)
            for p, o in zip(u.params, u.offsets):
                values[id(p)] = full[o:o + p.numel()].view(p.shape).clone()
        names = {n: p for n, p in self.model.named_parameters(remove_duplicate=False)}
        out = {}
        for k, v in self.model.state_dict().items():
            p = names.get(k)
            out[k] = values[id(p)] if p is not None and id(p) in values else v.detach().clone()
        return out

    @torch.no_grad()
    def load_full_state_dict(self, state: Dict[str, torch.Tensor], strict: bool = True) -> None:
        """Take this rank's pieces of a dense state dict."""
        names = {n: p for n, p in self.model.named_parameters(remove_duplicate=False)}
        place = {id(p): (u, o) for u in self.units for p, o in zip(u.params, u.offsets)}
        have = {id(p) for k, p in names.items() if k in state}
        missing = [k for k, p in names.items() if id(p) not in have]     # a tied weight may come under either name
        if strict and missing:
            raise KeyError(f"missing parameters: {missing[:4]}")
        if self._sym:
            self._sync.barrier()      # no peer is still gathering the pieces that are about to change
        for k, p in names.items():
            if k not in state:
                continue
            src = state[k].reshape(-1)
            if id(p) not in place:
                p.data.copy_(state[k].to(p.device, p.dtype))
                continue
            u, o = place[id(p)]
            g0 = self.rank * u.per                       # owned range in unit coordinates
            lo, hi = max(o, g0), min(o + p.numel(), g0 + u.per)
            if lo < hi:
                self.data[u.local + lo - g0:u.local + hi - g0].copy_(src[lo - o:hi - o].to(self.device, self.dtype))
        self.invalidate()
