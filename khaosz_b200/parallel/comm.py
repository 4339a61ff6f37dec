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
from typing import List, Optional

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


class GradReducer:
    """Owns the symmetric homes of an executor's flat buffers and the fused optimizer step."""

    fuses_optimizer = True
    gathers_params = True

    def __init__(self, flat: FlatParameters, mode: str, group=None):
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
        self.slice_off = self.rank * self.slice_n
        self._m = torch.zeros(self.slice_n, dtype=torch.float32, device=dev)
        self._v = torch.zeros(self.slice_n, dtype=torch.float32, device=dev)
        self._scratch = torch.zeros(2, dtype=torch.float32, device=dev)
        self._lr_dev = torch.zeros(2, dtype=torch.float32, device=dev)
        self.use_multicast = bool(self.params.multicast_ptr and self.grads.multicast_ptr)

    @classmethod
    def create(cls, flat: FlatParameters, mode: str = "allreduce", group=None) -> Optional["GradReducer"]:
        if not (flat.data.is_cuda and flat.data.dtype == torch.bfloat16 and _lib.has("kb_reduce_adamw")):
            return None
        ws = dist.get_world_size(group)
        if ws > 8 or flat.numel % (8 * ws):
            return None
        return cls(flat, mode, group)

    def reduce(self) -> None:
        """Gradient reduction is part of :meth:`fused_step`; nothing to do at backward time."""

    def allreduce_grads(self) -> None:
        """Stand-alone mean all-reduce of the gradient buffer (for optimizers that cannot fuse)."""
        allreduce_(self.grads, self.ctrl, 1.0 / self.ws, self.use_multicast)

    def fused_step(self, opt, lr, beta1, beta2, eps, wd, clip, step) -> None:
        _lib.set_device_floats(self._lr_dev, lr, step)   # launch arguments: no staging buffer to overwrite
        mc_g = ctypes.c_void_p(self.grads.multicast_ptr) if self.use_multicast else None
        mc_p = ctypes.c_void_p(self.params.multicast_ptr) if self.use_multicast else None
        check(lib().kb_reduce_adamw(self.grads.ptrs, self.params.ptrs, self.ctrl.flags.ptrs, self.ctrl.norms.ptrs,
                                    mc_g, mc_p, self.rank, self.ws, self.slice_off, self.slice_n, ptr(self._m),
                                    ptr(self._v), ptr(self._lr_dev), beta1, beta2, eps, wd, float(clip or 0.0),
                                    ptr(self._scratch), self.ctrl.next_epoch(), stream()), "reduce_adamw")
        _lib.add_launches(2)
        opt.last_grad_norm = self._scratch[1:2].sqrt()

    # optimizer-state plumbing used by FusedAdamW.state_dict / load_state_dict
    def moments(self):
        return self._m, self._v, (self.slice_off, self.slice_n)
