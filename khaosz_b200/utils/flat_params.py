"""Flat parameter / gradient storage.

All parameters of a model become views of one contiguous buffer (and, optionally, their
gradients views of a second one).  That gives:

* q/k/v and gate/up weights that are adjacent in memory, so each group runs as one GEMM;
* weight gradients accumulated by the GEMM epilogue straight into the flat gradient buffer
  (``param.main_grad``), with ``param.grad`` aliasing the same memory for optimizers, clipping
  and hooks;
* one-launch optimizer steps, gradient norms and collectives over the whole model.
"""

from __future__ import annotations

from typing import Dict, List, Optional

import torch
import torch.nn as nn

ALIGN_ELEMS = 8  # 16 bytes of bf16: TMA and 128-bit accesses need it


class FlatParameters:
    def __init__(self, model: nn.Module, with_grad: bool = True, buffer: Optional[torch.Tensor] = None,
                 grad_buffer: Optional[torch.Tensor] = None, pad_to: int = ALIGN_ELEMS):
        params: List[nn.Parameter] = []
        seen = set()
        for p in model.parameters():
            if id(p) not in seen:
                seen.add(id(p))
                params.append(p)
        if not params:
            raise ValueError("model has no parameters")
        dtype, device = params[0].dtype, params[0].device
        if any(p.dtype != dtype or p.device != device for p in params):
            raise ValueError("FlatParameters needs one dtype and one device for all parameters")
        self.params = params
        self.offsets: List[int] = []
        off = 0
        for p in params:
            off = (off + ALIGN_ELEMS - 1) // ALIGN_ELEMS * ALIGN_ELEMS
            self.offsets.append(off)
            off += p.numel()
        self.numel = (off + pad_to - 1) // pad_to * pad_to
        self.data = buffer if buffer is not None else torch.zeros(self.numel, dtype=dtype, device=device)
        assert self.data.numel() >= self.numel
        with torch.no_grad():
            for p, o in zip(params, self.offsets):
                view = self.data[o:o + p.numel()].view(p.shape)
                view.copy_(p.data)
                p.data = view
        self.grad: Optional[torch.Tensor] = None
        if with_grad:
            self.grad = grad_buffer if grad_buffer is not None else torch.zeros(self.numel, dtype=dtype, device=device)
            for p, o in zip(params, self.offsets):
                if p.requires_grad:
                    g = self.grad[o:o + p.numel()].view(p.shape)
                    p.main_grad = g
                    p.grad = g

    def rebind(self, data: torch.Tensor, grad: Optional[torch.Tensor] = None) -> None:
        """Move the storage to new buffers of the same layout (e.g. symmetric memory) and
        re-point every parameter / gradient view."""
        assert data.numel() >= self.numel and data.dtype == self.data.dtype
        with torch.no_grad():
            data[: self.numel].copy_(self.data[: self.numel])
            self.data = data
            for p, o in zip(self.params, self.offsets):
                p.data = data[o:o + p.numel()].view(p.shape)
            if grad is not None:
                if self.grad is not None:
                    grad[: self.numel].copy_(self.grad[: self.numel])
                self.grad = grad
                for p, o in zip(self.params, self.offsets):
                    if p.requires_grad:
                        g = grad[o:o + p.numel()].view(p.shape)
                        p.main_grad = g
                        p.grad = g

    def zero_grad(self) -> None:
        if self.grad is not None:
            self.grad.zero_()
            for p in self.params:
                if p.requires_grad and p.grad is None:
                    p.grad = p.main_grad

    def named_offsets(self, model: nn.Module) -> Dict[str, int]:
        ids = {id(p): o for p, o in zip(self.params, self.offsets)}
        return {n: ids[id(p)] for n, p in model.named_parameters()}
