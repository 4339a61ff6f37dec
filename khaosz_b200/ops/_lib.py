"""ctypes binding of the sm_100a kernel library.

The library is built in-tree (``khaosz_b200/ops/libkhaosz_b200_kernels.so``) by
``khaosz_b200.ops.build``.  Every wrapper in ``khaosz_b200.ops`` goes through :func:`lib`;
on a CUDA device a missing library is an error, never a silent fallback.
"""

from __future__ import annotations

import ctypes
import os
import threading
from ctypes import c_float, c_int, c_long, c_longlong, c_void_p
from pathlib import Path

import torch

_LIB = None
_LOCK = threading.Lock()
_LAUNCHES = 0  # number of kernel-library launches issued by this process

STATUS = {1: "bad argument (shape/alignment)", 2: "CUDA launch error", 3: "tensor-map encode error",
          4: "size beyond the supported maximum"}
DEVICE_ERR = {1: "timeout waiting for TMA data", 2: "timeout waiting for a free stage",
              3: "timeout waiting for the accumulator", 4: "timeout waiting for a free accumulator",
              5: "timeout waiting for a peer flag", 6: "timeout", 7: "bad argument on device"}


class KernelError(RuntimeError):
    pass


def lib_path() -> Path:
    return Path(__file__).resolve().parent / "libkhaosz_b200_kernels.so"


def _declare(lib):
    P, I, L, LL, F = c_void_p, c_int, c_long, c_longlong, c_float
    sigs = {
        "kb_last_error": ([], I),
        "kb_sm_count": ([], I),
        "kb_error_probe": ([P, P], I),
        "kb_store_f32x2": ([P, F, F, P], I),
        "kb_copy_async": ([P, P, LL, P], I),
        "kb_last_tmap_error": ([], I),
        "kb_gemm_bf16": ([P, P, P, P, I, I, I, L, L, L, L, I, I, I, P], I),
        "kb_gemm_bf16_bn": ([P, P, P, P, I, I, I, L, L, L, L, I, I, I, I, P], I),
        "kb_gemm_bf16_pair": ([P, P, P, P, I, I, I, L, L, L, L, I, I, I, P], I),
        "kb_gemm_bf16_pair_bn": ([P, P, P, P, I, I, I, L, L, L, L, I, I, I, I, P], I),
        "kb_gemm_swiglu_bf16": ([P, P, P, P, I, I, I, L, L, L, L, I, P], I),
        "kb_rmsnorm_fwd": ([P, P, P, P, P, P, I, I, F, P], I),
        "kb_rmsnorm_bwd_partials": ([I], I),
        "kb_rmsnorm_bwd": ([P, P, P, P, P, P, P, P, I, I, P], I),
        "kb_rope": ([P, P, P, P, I, I, I, I, L, I, P], I),
        "kb_swiglu_fwd": ([P, P, I, I, P], I),
        "kb_swiglu_bwd": ([P, P, P, I, I, P], I),
        "kb_ce_fwd": ([P, P, P, P, P, I, I, L, F, LL, P], I),
        "kb_ce_bwd": ([P, P, P, P, P, I, I, L, F, LL, I, P], I),
        "kb_embedding_fwd": ([P, P, P, I, I, I, P], I),
        "kb_embedding_bwd": ([P, P, P, I, I, I, P], I),
        "kb_sumsq_bf16": ([P, LL, P, P], I),
        "kb_adamw_bf16": ([P, P, P, P, LL, P, F, F, F, F, F, P, F, P], I),
        "kb_flash_fwd": ([P, P, P, P, P, I, I, I, I, I, L, L, L, L, F, I, P], I),
        "kb_flash_fwd_rect": ([P, P, P, P, P, I, I, I, I, I, I, L, L, L, L, F, I, P], I),
        "kb_flash_bwd": ([P, P, P, P, P, P, P, P, P, P, I, I, I, I, I, L, L, L, L, L, L, L, L, F, I, P], I),
        "kb_paged_decode_attn": ([P, P, P, P, P, P, P, P, I, I, I, I, I, I, I, L, L, F, P], I),
        "kb_paged_decode_tc": ([P, P, P, P, P, P, P, P, I, I, I, I, I, I, I, I, L, L, F, P], I),
        "kb_paged_kv_write": ([P, P, P, P, P, I, I, L, L, P], I),
        "kb_rope_norm_kvwrite": ([P, P, P, P, P, F, P, P, P, I, I, I, I, I, L, P], I),
        "kb_sample": ([P, P, P, P, P, P, I, I, L, LL, P], I),
        "kb_gemm_w8": ([P, P, P, P, I, I, I, L, L, L, P], I),
        "kb_quant_w8": ([P, P, P, I, I, P], I),
        "kb_quant_fp8_1x128": ([P, P, P, I, I, L, P], I),
        "kb_quant_fp8_128x128": ([P, P, P, I, I, L, P], I),
        "kb_gemm_fp8": ([P, P, P, P, P, I, I, I, L, L, L, P], I),
        "kb_comm_slots": ([], I),
        "kb_gemm_comm": ([P, P, P, P, P, P, I, I, I, L, L, L, L, I, I, I, I, I, I, I, ctypes.c_uint, P, I, P, ctypes.c_uint, P, I, P, P, P], I),
        "kb_reduce_adamw": ([P, P, P, P, P, P, I, I, LL, LL, P, P, P, F, F, F, F, F, P, ctypes.c_uint, P], I),
        "kb_reduce_bucket": ([P, P, P, I, I, LL, LL, I, I, P, ctypes.c_uint, I, I, P], I),
        "kb_adamw_buckets": ([P, P, P, P, P, I, I, LL, LL, P, P, P, F, F, F, F, F, P, ctypes.c_uint, P], I),
        "kb_allreduce_bf16": ([P, P, P, I, I, LL, F, ctypes.c_uint, P], I),
        "kb_reducescatter_bf16": ([P, P, P, I, I, LL, F, P, ctypes.c_uint, P], I),
        "kb_allgather_bf16": ([P, P, P, I, I, LL, ctypes.c_uint, P], I),
        "kb_broadcast_bf16": ([P, P, P, I, I, I, LL, ctypes.c_uint, P], I),
        "kb_unit_reduce_bf16": ([P, P, P, I, I, LL, F, P, I, ctypes.c_uint, I, I, P], I),
        "kb_peer_barrier": ([P, I, I, I, ctypes.c_uint, I, P], I),
        "kb_rmsnorm_bwd_static": ([P, P, P, P, P, P, P, I, I, P], I),
    }
    for name, (argtypes, restype) in sigs.items():
        fn = getattr(lib, name, None)
        if fn is not None:
            fn.argtypes = argtypes
            fn.restype = restype


def lib():
    """Load (building if needed) and return the kernel library."""
    global _LIB
    if _LIB is not None:
        return _LIB
    with _LOCK:
        if _LIB is not None:
            return _LIB
        path = lib_path()
        if os.environ.get("KHAOSZ_B200_NO_BUILD") != "1":
            from .build import ensure_built

            try:
                ensure_built()
            except Exception as exc:  # pragma: no cover - toolchain problems
                if not path.exists():
                    raise KernelError(f"kernel library is missing and cannot be built: {exc}") from exc
        if not path.exists():
            raise KernelError(f"kernel library not found at {path}")
        handle = ctypes.CDLL(str(path))
        _declare(handle)
        _LIB = handle
    return _LIB


def has(name: str) -> bool:
    return hasattr(lib(), name)


def available() -> bool:
    """True when CUDA kernels can run in this process (a GPU is visible)."""
    return torch.cuda.is_available()


def use_kernels(*tensors: torch.Tensor) -> bool:
    """Kernel path is taken for CUDA bf16 tensors; anything else is the torch oracle path."""
    t0 = tensors[0]
    return t0.is_cuda and t0.dtype == torch.bfloat16


def ptr(t):
    return None if t is None else c_void_p(t.data_ptr())


def stream():
    return c_void_p(torch.cuda.current_stream().cuda_stream)


def check(status: int, what: str):
    global _LAUNCHES
    _LAUNCHES += 1
    if status != 0:
        extra = f" (CUresult {lib().kb_last_tmap_error()})" if status == 3 else ""
        raise KernelError(f"{what}: {STATUS.get(status, status)}{extra}")


def launch_count() -> int:
    return _LAUNCHES


def add_launches(n: int):
    global _LAUNCHES
    _LAUNCHES += n


class ErrorProbe:
    """Non-blocking reads of the device error word.

    ``post()`` enqueues a 4-byte copy of the word into page-locked host memory plus an event on the
    current stream; ``poll()`` looks at the probes whose event has completed and raises for the first
    non-zero code.  Neither call waits for the device."""

    def __init__(self, slots: int = 8):
        self._host = torch.zeros(slots, dtype=torch.int32).pin_memory()
        self._pending = []      # (slot, event)
        self._free = list(range(slots))

    def post(self) -> None:
        if not self._free:
            return              # enough probes in flight; the next poll frees some
        slot = self._free.pop()
        dst = c_void_p(self._host.data_ptr() + 4 * slot)
        if lib().kb_error_probe(dst, stream()) != 0:
            self._free.append(slot)
            return
        ev = torch.cuda.Event()
        ev.record()
        self._pending.append((slot, ev))

    def poll(self, wait: bool = False) -> None:
        keep, code = [], 0
        for slot, ev in self._pending:
            if wait:
                ev.synchronize()
            if wait or ev.query():
                code = code or int(self._host[slot])
                self._free.append(slot)
            else:
                keep.append((slot, ev))
        self._pending = keep
        if code:
            lib().kb_last_error()   # clears the word
            raise KernelError(f"device-side kernel error: {DEVICE_ERR.get(code, code)}")


def set_device_floats(dst: torch.Tensor, a: float, b: float) -> None:
    """``dst[0], dst[1] = a, b`` on the current stream, the values carried as launch arguments."""
    check(lib().kb_store_f32x2(ptr(dst), float(a), float(b), stream()), "store_f32x2")
    add_launches(-1)


def raise_on_device_error():
    """Synchronising check of the device-side error word (bounded waits report here)."""
    code = lib().kb_last_error()
    if code != 0:
        raise KernelError(f"device-side kernel error: {DEVICE_ERR.get(code, code)}")
