"""Hand-written sm_100a kernels and their PyTorch-facing wrappers."""

from ._lib import KernelError, available, launch_count, raise_on_device_error
from .functional import (
    add_rms_norm,
    cross_entropy,
    cross_entropy_rows,
    embedding,
    fp8_linear_enabled,
    gemm,
    linear,
    linear_swiglu,
    multi_linear,
    rms_norm,
    rms_norm_fork,
    rope,
    rope_table,
    sdpa_reference,
    set_fp8_linear,
    swiglu,
    token_logprobs,
)

__all__ = [
    "KernelError", "available", "launch_count", "raise_on_device_error", "add_rms_norm", "cross_entropy",
    "cross_entropy_rows", "embedding", "gemm", "linear", "multi_linear", "rms_norm", "rope", "rope_table",
    "sdpa_reference", "swiglu", "linear_swiglu", "token_logprobs", "set_fp8_linear", "fp8_linear_enabled", "rms_norm_fork",
]
