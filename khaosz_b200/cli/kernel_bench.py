"""Micro-benchmark of one kernel family on one GPU (CUDA-event timing after warm-up, L2
flushed between timed launches).  Also the workload used for the committed ``ncu`` summaries:

    python -m khaosz_b200.cli.kernel_bench gemm --m 4096 --n 4096 --k 4096 --iters 3
    ncu --set full --clock-control none -k regex:gemm_bf16 -c 3 -o prof python -m khaosz_b200.cli.kernel_bench gemm ...
"""

from __future__ import annotations

import argparse
import json
import math

import torch

from .. import ops
from ..ops import attention as A


def _time(fn, iters: int, flush: torch.Tensor):
    fn()
    fn()
    torch.cuda.synchronize()
    total = 0.0
    for _ in range(iters):
        flush.zero_()  # evict the 126 MB L2
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        total += e0.elapsed_time(e1)
    return total / iters


def main(argv=None):
    p = argparse.ArgumentParser()
    p.add_argument("kernel", choices=["gemm", "gemm_pair", "gemm_swiglu", "gemm_w8", "gemm_fp8", "flash_fwd", "flash_bwd", "rmsnorm",
                                      "rmsnorm_bwd", "swiglu", "rope", "ce", "adamw", "decode", "sample", "embedding"])
    p.add_argument("--m", type=int, default=4096)
    p.add_argument("--n", type=int, default=4096)
    p.add_argument("--k", type=int, default=4096)
    p.add_argument("--batch", type=int, default=2)
    p.add_argument("--seq", type=int, default=2048)
    p.add_argument("--heads", type=int, default=16)
    p.add_argument("--kv_heads", type=int, default=4)
    p.add_argument("--iters", type=int, default=5)
    a = p.parse_args(argv)
    dev = "cuda"
    bf = torch.bfloat16
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=dev)
    M, N, K = a.m, a.n, a.k
    flops = bytes_ = 0.0
    if a.kernel in ("gemm", "gemm_pair"):
        x, w = torch.randn(M, K, device=dev, dtype=bf), torch.randn(N, K, device=dev, dtype=bf)
        out = torch.empty(M, N, device=dev, dtype=bf)
        if a.kernel == "gemm":
            from ..ops._lib import lib, ptr, stream

            fn = lambda: lib().kb_gemm_bf16(ptr(x), ptr(w), ptr(out), None, M, N, K, K, K, N, 0, 0, 0, 0, stream())
        else:
            from ..ops._lib import lib, ptr, stream

            fn = lambda: lib().kb_gemm_bf16_pair(ptr(x), ptr(w), ptr(out), None, M, N, K, K, K, N, 0, 0, 0, 0, stream())
        flops, bytes_ = 2.0 * M * N * K, 2.0 * (M * K + N * K + M * N)
    elif a.kernel == "gemm_swiglu":
        # gate|up projection with the SwiGLU epilogue: --n is the number of features F (the GEMM is 2F wide)
        from ..ops._lib import lib, ptr, stream

        x, w = torch.randn(M, K, device=dev, dtype=bf), torch.randn(2 * N, K, device=dev, dtype=bf) * 0.02
        gu, h = torch.empty(M, 2 * N, device=dev, dtype=bf), torch.empty(M, N, device=dev, dtype=bf)
        fn = lambda: lib().kb_gemm_swiglu_bf16(ptr(x), ptr(w), ptr(gu), ptr(h), M, N, K, K, K, 2 * N, N, 0, stream())
        flops, bytes_ = 4.0 * M * N * K, 2.0 * (M * K + 2 * N * K + 3 * M * N)
    elif a.kernel == "gemm_w8":
        from ..ops.quant import linear_w8, quantize_w8

        x, w = torch.randn(M, K, device=dev, dtype=bf), torch.randn(N, K, device=dev, dtype=bf) * 0.05
        q, s = quantize_w8(w)
        fn = lambda: linear_w8(x, q, s)
        flops, bytes_ = 2.0 * M * N * K, 2.0 * M * K + N * K + 2.0 * M * N
    elif a.kernel == "gemm_fp8":
        from ..ops import quant

        x, w = torch.randn(M, K, device=dev, dtype=bf), torch.randn(N, K, device=dev, dtype=bf) * 0.05
        a8, sa = quant.quantize_fp8_1x128(x)
        b8, sb = quant.quantize_fp8_128x128(w)
        fn = lambda: quant.gemm_fp8(a8, sa, b8, sb)
        flops, bytes_ = 2.0 * M * N * K, M * K + N * K + 2.0 * M * N
    elif a.kernel in ("flash_fwd", "flash_bwd"):
        B, S, H, Hkv, D = a.batch, a.seq, a.heads, a.kv_heads, 128
        qkv = torch.randn(B, S, H + 2 * Hkv, D, device=dev, dtype=bf)
        q, k, v = qkv[:, :, :H], qkv[:, :, H:H + Hkv], qkv[:, :, H + Hkv:]
        scale = 1 / math.sqrt(D)
        o, lse = A._flash_fwd(q, k, v, True, scale)
        if a.kernel == "flash_fwd":
            fn = lambda: A._flash_fwd(q, k, v, True, scale)
            flops = 4.0 * B * H * S * S * D / 2
        else:
            do = torch.randn_like(o)
            dqkv = torch.empty_like(qkv)
            fn = lambda: A._flash_bwd(q, k, v, o, do, lse, dqkv[:, :, :H], dqkv[:, :, H:H + Hkv], dqkv[:, :, H + Hkv:],
                                      True, scale)
            flops = 2.5 * 4.0 * B * H * S * S * D / 2
        bytes_ = 2.0 * qkv.numel() * 2
    elif a.kernel in ("rmsnorm", "rmsnorm_bwd"):
        x = torch.randn(M, N, device=dev, dtype=bf, requires_grad=True)
        w = torch.ones(N, device=dev, dtype=bf, requires_grad=True)
        if a.kernel == "rmsnorm":
            fn = lambda: ops.rms_norm(x.detach(), w.detach(), 1e-5)
            bytes_ = 2.0 * M * N * 2
        else:
            y = ops.rms_norm(x, w, 1e-5)
            g = torch.randn_like(y)
            fn = lambda: torch.autograd.grad(y, (x, w), g, retain_graph=True)
            bytes_ = 3.0 * M * N * 2
    elif a.kernel == "swiglu":
        gu = torch.randn(M, 2 * N, device=dev, dtype=bf)
        fn = lambda: ops.swiglu(gu)
        bytes_ = 3.0 * M * N * 2
    elif a.kernel == "rope":
        x = torch.randn(a.batch, a.seq, a.heads, 128, device=dev, dtype=bf)
        cs = ops.rope_table(128, a.seq, device=dev)
        fn = lambda: ops.rope(x, cs)
        bytes_ = 2.0 * x.numel() * 2
    elif a.kernel == "ce":
        logits = torch.randn(M, N, device=dev, dtype=bf)
        t = torch.randint(0, N, (M,), device=dev)
        fn = lambda: ops.cross_entropy(logits, t, 0.05)
        bytes_ = 2.0 * M * N
    elif a.kernel == "adamw":
        from ..ops._lib import lib, ptr, stream

        n = M * N
        pp, g = torch.randn(n, device=dev, dtype=bf), torch.randn(n, device=dev, dtype=bf)
        m, v = torch.zeros(n, device=dev), torch.zeros(n, device=dev)
        lr = torch.tensor([1e-3, 1.0], device=dev)
        fn = lambda: lib().kb_adamw_bf16(ptr(pp), ptr(g), ptr(m), ptr(v), n, ptr(lr), 0.9, 0.95, 1e-8, 0.01, 1.0, None,
                                         0.0, stream())
        bytes_ = n * (2 + 2 + 2 + 16.0)
    elif a.kernel == "decode":
        from ..inference import KVCache

        B, H, Hkv, page = a.batch, a.heads, a.kv_heads, 16
        kv = KVCache(1, B * (a.seq // page + 2), page, Hkv, 128, dev, bf)
        names = [f"s{i}" for i in range(B)]
        for nme in names:
            kv.task_alloc(nme, list(range(a.seq)))
        table = kv.make_table_tensor(names, dev)
        lens = torch.full((B,), a.seq, device=dev)
        q = torch.randn(B, 1, H, 128, device=dev, dtype=bf)
        kn, vn = torch.randn(B, 1, Hkv, 128, device=dev, dtype=bf), torch.randn(B, 1, Hkv, 128, device=dev, dtype=bf)
        view = kv.bind(table, seq_lens=lens)
        fn = lambda: view.attention(0, q, kn, vn)
        bytes_ = 2.0 * B * a.seq * Hkv * 128 * 2
    elif a.kernel == "sample":
        from ..inference.sample import fused_sample

        logits = torch.randn(M, 32000, device=dev, dtype=bf)
        fn = lambda: fused_sample(logits, 0.8, 50, 0.95)
        bytes_ = 2.0 * M * 32000
    else:
        table = torch.randn(32000, N, device=dev, dtype=bf)
        ids = torch.randint(0, 32000, (M,), device=dev)
        fn = lambda: ops.embedding(ids, table)
        bytes_ = 2.0 * M * N * 2
    ms = _time(fn, a.iters, flush)
    ops.raise_on_device_error()
    row = {"kernel": a.kernel, "ms": ms}
    if flops:
        row["tflops"] = flops / ms / 1e9
    if bytes_:
        row["gbps"] = bytes_ / ms / 1e6
    print(json.dumps(row))


if __name__ == "__main__":
    main()
