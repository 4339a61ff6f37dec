"""Tensor parallelism with sequence-sharded activations (Megatron style) on fused kernels.

Between tensor-parallel regions activations are sharded over the token dimension.  A
column-parallel layer consumes them through **all-gather -> GEMM** (a copier warp in every CTA
pulls the peers' token shards once over NVLink into a local image while the tiles of the local
shard are already being multiplied; the image is kept for the weight gradient), a row-parallel
layer hands its partial sums back through **GEMM -> reduce-scatter** (training) or
**GEMM -> all-reduce** (decode); the backward pass runs on the same kernel with MN-major
operands.  The kernels take their barrier epoch from device memory, so a step that contains
them can be recorded into a CUDA graph.  On CPU (gloo) the same modules fall back to
``torch.distributed`` collectives, which is also the numerical reference in the tests.

The reference only ships forward-only ``ColumnParallelLinear`` / ``RowParallelLinear``
primitives (``astrai/parallel/module.py:18-115``); the class names, weight shapes and the
``load_state_dict`` slicing of a full weight are kept.
"""

from __future__ import annotations

import ctypes
from typing import Dict, Optional, Tuple

import torch
import torch.distributed as dist
import torch.nn as nn

from ..ops import _lib
from ..ops._lib import check, lib, ptr, stream
from .comm import PeerControl, SymmetricBuffer


class TPContext:
    """Per-process state of the fused tensor-parallel kernels: control flags, a pool of
    symmetric activation / staging buffers and the grid-barrier words."""

    _current: Optional["TPContext"] = None

    def __init__(self, group=None, device=None):
        self.group = group if group is not None else dist.group.WORLD
        self.ws = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        self.device = device if device is not None else torch.device("cuda", torch.cuda.current_device())
        self.use_kernels = self.device.type == "cuda" and self.ws > 1 and self.ws <= 8 and _lib.has("kb_gemm_comm")
        self._pool: Dict[Tuple[str, int], SymmetricBuffer] = {}
        self._images: Dict[Tuple[str, int, int, int], list] = {}
        self._turns: Dict[Tuple[str, int, int], int] = {}
        self._retired: list = []
        if self.use_kernels:
            self.ctrl = PeerControl(self.device, self.group)
            self.grid_sync = torch.zeros(2, dtype=torch.int32, device=self.device)
            # The barrier epoch of the fused kernels lives on the device (advanced by a one-thread
            # kernel behind every launch), so that a captured CUDA graph can be replayed; every
            # rank starts at the same value and issues the same sequence of fused kernels.
            self.epoch_dev = torch.full((1,), 4, dtype=torch.int32, device=self.device)

    @classmethod
    def get(cls, group=None) -> "TPContext":
        if cls._current is None:
            dev = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")
            cls._current = cls(group, dev)
        return cls._current

    @classmethod
    def reset(cls) -> None:
        cls._current = None

    def buffer(self, tag: str, numel: int, grow: bool = False) -> SymmetricBuffer:
        """Symmetric bf16 buffer of at least ``numel`` elements (collective on first use per tag/size).
        ``grow=True`` keeps one buffer per tag and replaces it by a larger one (next power of two)
        only when needed: for scratch whose size follows the batch (staging of the reduced output),
        so that a new batch size does not cost a new symmetric allocation."""
        if grow:
            buf = self._pool.get((tag, -1))
            if buf is None or buf.tensor.numel() < numel:
                if buf is not None:
                    self._retired.append(buf)  # recorded CUDA graphs may still point at it
                cap = 1 << max(int(numel - 1).bit_length(), 16)
                buf = SymmetricBuffer(cap, torch.bfloat16, self.device, self.group, zero=True)
                torch.cuda.synchronize(self.device)
                dist.barrier(group=self.group)
                self._pool[(tag, -1)] = buf
            return buf
        key = (tag, numel)
        buf = self._pool.get(key)
        if buf is None:
            buf = SymmetricBuffer(numel, torch.bfloat16, self.device, self.group, zero=True)
            torch.cuda.synchronize(self.device)
            dist.barrier(group=self.group)
            self._pool[key] = buf
        return buf

    def gather_image(self, tag: str, shard: torch.Tensor):
        """Symmetric image of a whole row-sharded operand with this rank's shard copied into its
        rows.  Returns ``(buffer, ready_counters, ready_target)`` for the copy-mode gather of the
        fused kernel (peers pull the other shards inside the kernel)."""
        rows, cols = shard.shape
        # two images per tag, used alternately: a peer may still be reading the image of the
        # previous call when this rank prepares the next one (the kernel has no exit barrier)
        turn = self._turns.get((tag, rows, cols), 0)
        self._turns[(tag, rows, cols)] = turn ^ 1
        key = (tag, rows, cols, turn)
        entry = self._images.get(key)
        if entry is None:
            buf = self.buffer(f"{tag}.img{turn}", self.ws * rows * cols)
            # one arrival counter per 128-row chunk + (last word) the number of copy-mode calls so far
            ready = torch.zeros(self.ws * rows // 128 + 1, dtype=torch.int32, device=self.device)
            entry = self._images[key] = [buf, ready, 0]
        buf, ready, calls = entry
        buf.tensor[: self.ws * rows * cols].view(self.ws * rows, cols)[self.rank * rows:(self.rank + 1) * rows].copy_(shard)
        entry[2] = calls + 1
        pieces_per_chunk = (128 * cols * 2 + 16383) // 16384
        return buf, ready, entry[2] * pieces_per_chunk

    def stage_in(self, tag: str, t: torch.Tensor) -> SymmetricBuffer:
        """Copy a local tensor into symmetric memory so that peers can read it (two buffers per
        tag, used alternately, for the same reason as in ``gather_image``)."""
        turn = self._turns.get((tag, t.numel(), -1), 0)
        self._turns[(tag, t.numel(), -1)] = turn ^ 1
        buf = self.buffer(f"{tag}.{turn}", t.numel())
        buf.tensor[: t.numel()].view(t.shape).copy_(t)
        return buf


def _ptr_list(values):
    return (ctypes.c_void_p * len(values))(*values)


def _comm_gemm(ctx: TPContext, a, b, *, a_mn=False, b_mn=False, a_gather=False, b_gather=False, c_mode=0,
               tag="tp", trace: Optional[torch.Tensor] = None, want_image: bool = False):
    """``op(A) op(B)^T`` with the fused collective.  ``a`` / ``b`` are local tensors (gathered
    operands are this rank's shard).  Returns the local result (c_mode 0), this rank's rows of the
    sum (c_mode 1) or the full sum (c_mode 2).  ``trace`` (int64 [6], device) receives CTA 0's
    timestamps: entered, all ranks entered, own tiles done, all CTAs done, all ranks done, reduced.
    ``want_image=True`` returns ``(result, image)`` where ``image`` is the local copy of the whole
    gathered operand that the kernel assembled (``None`` when the direct mode ran); it stays valid
    until the second-next call with the same tag and shape."""
    ws, rank = ctx.ws, ctx.rank
    a_rows, a_cols = a.shape
    b_rows, b_cols = b.shape
    A_rows = a_rows * ws if a_gather else a_rows
    B_rows = b_rows * ws if b_gather else b_rows
    M = a_cols if a_mn else A_rows
    K = A_rows if a_mn else a_cols
    N = b_cols if b_mn else B_rows
    Kb = B_rows if b_mn else b_cols
    assert K == Kb, (K, Kb)
    copy, ready, ready_target, calls_dev = 0, None, 0, None
    if (a_gather and a_rows % 128 == 0) or (b_gather and b_rows % 128 == 0):
        copy = 1  # whole 128-row chunks: peers' shards are pulled once into a local image
    image = None
    if a_gather and copy:
        sa, ready, ready_target = ctx.gather_image(tag + ".a", a)
        a_ptrs, lda = sa.ptrs, a_cols
        image = sa.tensor[: ws * a_rows * a_cols].view(ws * a_rows, a_cols)
    elif a_gather:
        sa = ctx.stage_in(tag + ".a", a)
        a_ptrs, lda = sa.ptrs, a_cols
    else:
        a = a if a.stride(-1) == 1 else a.contiguous()
        a_ptrs, lda = _ptr_list([a.data_ptr()] * ws), a.stride(0)
    if b_gather and copy:
        sb, ready, ready_target = ctx.gather_image(tag + ".b", b)
        b_ptrs, ldb = sb.ptrs, b_cols
        image = sb.tensor[: ws * b_rows * b_cols].view(ws * b_rows, b_cols)
    elif b_gather:
        sb = ctx.stage_in(tag + ".b", b)
        b_ptrs, ldb = sb.ptrs, b_cols
    else:
        b = b if b.stride(-1) == 1 else b.contiguous()
        b_ptrs, ldb = _ptr_list([b.data_ptr()] * ws), b.stride(0)
    c_local = out = None
    stage_ptrs = None
    if c_mode == 0:
        c_local = torch.empty((M, N), dtype=a.dtype, device=a.device)
        ldc, ldo = N, 0
    else:
        rows = M // ws if c_mode == 1 else M
        slot_rows = (rows + 127) // 128 * 128
        stage = ctx.buffer(tag + ".stage", ws * slot_rows * N, grow=True)
        stage_ptrs = stage.ptrs
        out = torch.empty((rows, N), dtype=a.dtype, device=a.device)
        ldc, ldo = N, N
    if ready is not None:
        calls_dev = ctypes.c_void_p(ready.data_ptr() + 4 * (ready.numel() - 1))
    check(lib().kb_gemm_comm(a_ptrs, b_ptrs, ptr(c_local), stage_ptrs, ctx.ctrl.flags.ptrs, ptr(out), M, N, K, lda, ldb,
                             ldc, ldo, int(a_mn), int(b_mn), int(a_gather), int(b_gather), c_mode, rank, ws,
                             0, ptr(ctx.grid_sync), copy, ptr(ready), ready_target, ptr(trace), 0, ptr(ctx.epoch_dev), calls_dev, stream()),
          "gemm_comm")
    result = c_local if c_mode == 0 else out
    return (result, image) if want_image else result


# ---- reference collectives (CPU/gloo and the oracle of the GPU tests) -----------------------
def _all_gather_rows(x: torch.Tensor, group) -> torch.Tensor:
    parts = [torch.empty_like(x) for _ in range(dist.get_world_size(group))]
    dist.all_gather(parts, x.contiguous(), group=group)
    return torch.cat(parts, dim=0)


def _reduce_scatter_rows(x: torch.Tensor, group) -> torch.Tensor:
    ws, rank = dist.get_world_size(group), dist.get_rank(group)
    x = x.contiguous()
    dist.all_reduce(x, group=group)
    n = x.shape[0] // ws
    return x[rank * n:(rank + 1) * n].clone()


def _kernel_ok(ctx: TPContext, *tensors) -> bool:
    return ctx.use_kernels and all(t.is_cuda and t.dtype == torch.bfloat16 for t in tensors)


class _ColumnParallelFn(torch.autograd.Function):
    """y[M, N_local] = all_gather(x_shard)[M, K] @ W_local[N_local, K]^T"""

    @staticmethod
    def forward(ctx, x_shard, w, tp):
        ctx.tp = tp
        ctx.full_x = None
        if _kernel_ok(tp, x_shard, w) and x_shard.shape[0] % 128 == 0:
            # the image of the gathered input assembled by the kernel is kept for the weight
            # gradient (one image pair per layer: the tag carries the weight's identity), so the
            # backward pass needs no second gather
            y, full_x = _comm_gemm(tp, x_shard, w, a_gather=True, tag=f"col.fwd.{id(w)}", want_image=True)
            ctx.full_x = full_x
            ctx.save_for_backward(x_shard if full_x is None else x_shard.new_empty(0), w)
            return y
        ctx.save_for_backward(x_shard, w)
        return _all_gather_rows(x_shard, tp.group) @ w.t()

    @staticmethod
    def backward(ctx, dy):
        x_shard, w = ctx.saved_tensors
        tp = ctx.tp
        dy = dy.contiguous()
        if ctx.full_x is not None:
            from ..ops.functional import gemm

            dx = _comm_gemm(tp, dy, w, b_mn=True, c_mode=1, tag="col.dx")                   # RS(dy W)
            dw = gemm(dy, ctx.full_x, a_mn=True, b_mn=True)                                  # dy^T AG(x), local
        elif _kernel_ok(tp, dy, w) and x_shard.shape[0] % 128 == 0:
            dx = _comm_gemm(tp, dy, w, b_mn=True, c_mode=1, tag="col.dx")                   # RS(dy W)
            dw = _comm_gemm(tp, dy, x_shard, a_mn=True, b_mn=True, b_gather=True, tag="col.dw")  # dy^T AG(x)
        else:
            dx = _reduce_scatter_rows(dy @ w, tp.group)
            dw = dy.t() @ _all_gather_rows(x_shard, tp.group)
        return dx, dw, None


class _RowParallelFn(torch.autograd.Function):
    """y_shard[M / ws, N] = reduce_scatter(x[M, K_local] @ W_local[N, K_local]^T)"""

    @staticmethod
    def forward(ctx, x, w, tp, all_reduce):
        ctx.tp, ctx.all_reduce = tp, all_reduce
        ctx.save_for_backward(x, w)
        x = x.contiguous()
        if _kernel_ok(tp, x, w) and (all_reduce or (x.shape[0] % (128 * tp.ws) == 0)):
            return _comm_gemm(tp, x, w, c_mode=2 if all_reduce else 1, tag="row.fwd")
        y = x @ w.t()
        if all_reduce:
            dist.all_reduce(y, group=tp.group)
            return y
        return _reduce_scatter_rows(y, tp.group)

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        tp = ctx.tp
        dy = dy.contiguous()
        if ctx.all_reduce:  # dy is already complete on every rank
            return dy @ w, dy.t() @ x, None, None
        if _kernel_ok(tp, dy, w) and dy.shape[0] % 128 == 0:
            from ..ops.functional import gemm

            dx, full_dy = _comm_gemm(tp, dy, w, a_gather=True, b_mn=True, tag="row.dx", want_image=True)  # AG(dy) W
            if full_dy is not None:   # the gathered dy is already in local memory
                dw = gemm(full_dy, x, a_mn=True, b_mn=True)                                          # AG(dy)^T x
            else:
                dw = _comm_gemm(tp, dy, x, a_mn=True, b_mn=True, a_gather=True, tag="row.dw")
        else:
            full = _all_gather_rows(dy, tp.group)
            dx, dw = full @ w, full.t() @ x
        return dx, dw, None, None


class _ShardedWeightFn(torch.autograd.Function):
    """``y = x @ all_gather(W_shard)^T`` for a weight whose rows are sharded over data-parallel
    ranks (fully sharded data parallel).  Forward and ``dx`` gather the weight inside the GEMM;
    ``dW`` is the GEMM -> reduce-scatter of ``dy^T x``, so every rank receives the rank-summed
    gradient of exactly the rows it owns."""

    @staticmethod
    def forward(ctx, x, w_shard, tp):
        ctx.tp = tp
        ctx.save_for_backward(x, w_shard)
        if _kernel_ok(tp, x, w_shard) and w_shard.shape[0] % 128 == 0:
            return _comm_gemm(tp, x, w_shard, b_gather=True, tag="fs.fwd")
        return x @ _all_gather_rows(w_shard, tp.group).t()

    @staticmethod
    def backward(ctx, dy):
        x, w_shard = ctx.saved_tensors
        tp = ctx.tp
        dy = dy.contiguous()
        if _kernel_ok(tp, dy, w_shard) and w_shard.shape[0] % 128 == 0:
            dx = _comm_gemm(tp, dy, w_shard, b_mn=True, b_gather=True, tag="fs.dx")   # dy AG(W)
            dw = _comm_gemm(tp, dy, x, a_mn=True, b_mn=True, c_mode=1, tag="fs.dw")    # RS(dy^T x)
        else:
            dx = dy @ _all_gather_rows(w_shard, tp.group)
            dw = _reduce_scatter_rows(dy.t() @ x, tp.group)
        return dx, dw, None


def sharded_weight_linear(x: torch.Tensor, w_shard: torch.Tensor, tp: "TPContext") -> torch.Tensor:
    shape = x.shape
    y = _ShardedWeightFn.apply(x.reshape(-1, shape[-1]), w_shard, tp)
    return y.view(*shape[:-1], y.shape[-1])


def _shard(full: torch.Tensor, dim: int, rank: int, ws: int) -> torch.Tensor:
    n = full.shape[dim] // ws
    return full.narrow(dim, rank * n, n).contiguous()


class ColumnParallelLinear(nn.Module):
    """Weight ``[out / ws, in]``.  Input: this rank's token shard ``[tokens / ws, in]`` (gathered
    inside the GEMM) or, with ``sequence_parallel=False``, the full replicated input.
    ``gather_output`` concatenates the output slices of all ranks (reference behaviour)."""

    def __init__(self, in_features: int, out_features: int, bias: bool = False, gather_output: bool = False,
                 sequence_parallel: bool = True, group=None):
        super().__init__()
        self.group = group
        self.ws = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        assert out_features % self.ws == 0
        self.in_features, self.out_features = in_features, out_features
        self.gather_output, self.sequence_parallel = gather_output, sequence_parallel
        self.weight = nn.Parameter(torch.empty(out_features // self.ws, in_features))
        self.bias = nn.Parameter(torch.zeros(out_features // self.ws)) if bias else None
        nn.init.normal_(self.weight, std=0.02)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        shape = x.shape
        x2 = x.reshape(-1, shape[-1])
        if self.ws == 1:
            y = x2 @ self.weight.t()
        elif self.sequence_parallel:
            y = _ColumnParallelFn.apply(x2, self.weight, TPContext.get(self.group))
        else:
            y = x2 @ self.weight.t()
        if self.bias is not None:
            y = y + self.bias
        if self.gather_output and self.ws > 1:
            parts = [torch.empty_like(y) for _ in range(self.ws)]
            dist.all_gather(parts, y.contiguous(), group=self.group)
            y = torch.cat(parts, dim=-1)
        return y

    def load_state_dict(self, state_dict, strict: bool = True, assign: bool = False):
        sd = dict(state_dict)
        w = sd.get("weight")
        if w is not None and w.shape[0] == self.out_features and self.ws > 1:
            sd["weight"] = _shard(w, 0, self.rank, self.ws)
            if "bias" in sd and sd["bias"].shape[0] == self.out_features:
                sd["bias"] = _shard(sd["bias"], 0, self.rank, self.ws)
        return super().load_state_dict(sd, strict=strict, assign=assign)


class RowParallelLinear(nn.Module):
    """Weight ``[out, in / ws]``.  Output: this rank's token shard of the summed result
    (``reduce_scatter=True``, sequence parallel) or the full sum on every rank."""

    def __init__(self, in_features: int, out_features: int, bias: bool = False, reduce_scatter: bool = True,
                 group=None):
        super().__init__()
        self.group = group
        self.ws = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        assert in_features % self.ws == 0
        self.in_features, self.out_features, self.reduce_scatter = in_features, out_features, reduce_scatter
        self.weight = nn.Parameter(torch.empty(out_features, in_features // self.ws))
        self.bias = nn.Parameter(torch.zeros(out_features)) if bias else None
        nn.init.normal_(self.weight, std=0.02)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        x2 = x.reshape(-1, x.shape[-1])
        if self.ws == 1:
            y = x2 @ self.weight.t()
        else:
            y = _RowParallelFn.apply(x2, self.weight, TPContext.get(self.group), not self.reduce_scatter)
        return y if self.bias is None else y + self.bias

    def load_state_dict(self, state_dict, strict: bool = True, assign: bool = False):
        sd = dict(state_dict)
        w = sd.get("weight")
        if w is not None and w.shape[1] == self.in_features and self.ws > 1:
            sd["weight"] = _shard(w, 1, self.rank, self.ws)
        return super().load_state_dict(sd, strict=strict, assign=assign)
