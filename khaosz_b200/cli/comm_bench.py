"""Benchmark of the fused compute+collective kernels against "library collective, then GEMM".

Run one process per GPU::

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 \
        --master-port 29611 -m khaosz_b200.cli.comm_bench --tokens 8192

Every case is timed on the device with CUDA events after warm-up, the reported time is the
maximum over ranks, and each fused kernel is given as a fraction of its roofline: the slower of
(FLOPs / GEMM peak) and (bytes that must cross NVLink per GPU / link bandwidth).  Shapes are the
tensor-parallel linears of the 1B decoder (d_model 2048, ffn 5632) at ``--tokens`` tokens.
"""

from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist


def _timed(fn, iters: int, warmup: int = 3) -> float:
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) / iters], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return t.item()


def main(argv=None) -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--tokens", type=int, default=8192)
    ap.add_argument("--dim", type=int, default=2048)
    ap.add_argument("--ffn", type=int, default=5632)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--gemm_peak_tflops", type=float, default=1399.5, help="measured sustained bf16 GEMM peak")
    ap.add_argument("--link_gbs", type=float, default=770.0, help="measured peer copy bandwidth per direction")
    ap.add_argument("--nvls", type=int, default=1)
    ap.add_argument("--model_params", type=int, default=1_148_000_000, help="length of the optimizer-step buffer")
    ap.add_argument("--unit_numel", type=int, default=45_092_864, help="parameters of one decoder block (full-shard rows)")
    ap.add_argument("--only", default="", help="comma-separated groups to run: tp, collectives, unit, optimizer (default: all)")
    args = ap.parse_args(argv)

    rank, ws = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if not args.nvls:
        os.environ["KHAOSZ_B200_NVLS"] = "0"
    dist.init_process_group("nccl", device_id=dev)

    from .. import ops
    from ..ops import raise_on_device_error
    from ..parallel.comm import PeerControl, SymmetricBuffer, allreduce_
    from ..parallel.tensor_parallel import TPContext, _comm_gemm

    tp = TPContext.get()
    T, d, f = args.tokens, args.dim, args.ffn
    gen = torch.Generator(device=dev).manual_seed(rank)

    def rnd(*shape):
        return (torch.randn(*shape, device=dev, generator=gen) * 0.05).to(torch.bfloat16)

    results = []
    trace = torch.zeros(6, dtype=torch.int64, device=dev)
    groups = {g for g in args.only.split(",") if g} or {"tp", "collectives", "unit", "optimizer"}

    def phases(fn):
        """One extra launch with CTA 0's phase timestamps (microseconds between the marks)."""
        trace.zero_()
        fn(trace)
        torch.cuda.synchronize()
        t = trace.tolist()
        names = ["wait_all_ranks_entered", "own_tiles_and_copies", "wait_all_ctas", "wait_all_ranks_done", "reduce"]
        return {n: round((t[i + 1] - t[i]) / 1e3, 1) for i, n in enumerate(names) if t[i + 1] and t[i]}

    def report(name, fused_ms, base_ms, flops, link_bytes, phase=None):
        t_flop = flops / (args.gemm_peak_tflops * 1e12) * 1e3
        t_link = link_bytes / (args.link_gbs * 1e9) * 1e3
        roof = max(t_flop, t_link)
        results.append({"case": name, "fused_ms": round(fused_ms, 4), "library_ms": round(base_ms, 4),
                        "speedup": round(base_ms / fused_ms, 3), "roofline_ms": round(roof, 4),
                        "bound": "tensor" if t_flop >= t_link else "nvlink",
                        "fraction_of_roofline": round(roof / fused_ms, 3), "phases_us": phase})

    if "tp" in groups:
        # ---- all-gather -> GEMM (column parallel gate|up): [T/ws, d] shards x W[2f/ws, d]
        n_loc = (2 * f // ws) // 8 * 8
        x_shard, w_col = rnd(T // ws, d), rnd(n_loc, d)
        full = torch.empty(T, d, dtype=torch.bfloat16, device=dev)

        def ag_fused(tr=None):
            return _comm_gemm(tp, x_shard, w_col, a_gather=True, tag="bench.col", trace=tr)

        def ag_lib():
            dist.all_gather_into_tensor(full, x_shard)
            return ops.gemm(full, w_col)

        report("all_gather->gemm (gate|up)", _timed(ag_fused, args.iters), _timed(ag_lib, args.iters),
               2.0 * T * n_loc * d, (ws - 1) / ws * T * d * 2, phases(ag_fused))

        # ---- GEMM -> reduce-scatter (row parallel down): x[T, f/ws] x W[d, f/ws] -> rows T/ws
        k_loc = (f // ws) // 8 * 8
        x_row, w_row = rnd(T, k_loc), rnd(d, k_loc)
        rs_out = torch.empty(T // ws, d, dtype=torch.bfloat16, device=dev)

        def rs_fused(tr=None):
            return _comm_gemm(tp, x_row, w_row, c_mode=1, tag="bench.row", trace=tr)

        def rs_lib():
            dist.reduce_scatter_tensor(rs_out, ops.gemm(x_row, w_row))
            return rs_out

        report("gemm->reduce_scatter (down)", _timed(rs_fused, args.iters), _timed(rs_lib, args.iters),
               2.0 * T * d * k_loc, (ws - 1) / ws * T * d * 2, phases(rs_fused))

        # ---- GEMM -> all-reduce (decode, 256 tokens)
        Td = 256
        xd = rnd(Td, k_loc)

        def ar_fused(tr=None):
            return _comm_gemm(tp, xd, w_row, c_mode=2, tag="bench.dec", trace=tr)

        def ar_lib():
            y = ops.gemm(xd, w_row)
            dist.all_reduce(y)
            return y

        report("gemm->all_reduce (decode, 256 tokens)", _timed(ar_fused, args.iters), _timed(ar_lib, args.iters),
               2.0 * Td * d * k_loc, 2 * (ws - 1) / ws * Td * d * 2, phases(ar_fused))

    if "collectives" in groups:
        # ---- stand-alone all-reduce of a 256 MiB gradient bucket
        n = 128 * 1024 * 1024
        buf = SymmetricBuffer(n, torch.bfloat16, dev)
        ctrl = PeerControl(dev)
        buf.tensor.normal_(generator=gen)
        plain = buf.tensor.clone()
        torch.cuda.synchronize()
        dist.barrier()
        report("all_reduce 256 MiB (kernel vs NCCL)", _timed(lambda: allreduce_(buf, ctrl, scale=1.0 / ws), args.iters),
               _timed(lambda: dist.all_reduce(plain), args.iters), 0.0, 2 * (ws - 1) / ws * n * 2)

        # ---- stand-alone reduce-scatter / all-gather / broadcast of the same buffer against NCCL
        from ..parallel.comm import all_gather_, broadcast_, reduce_scatter

        piece = torch.empty(n // ws, dtype=torch.bfloat16, device=dev)
        report("reduce_scatter 256 MiB (kernel vs NCCL)", _timed(lambda: reduce_scatter(buf, ctrl, out=piece), args.iters),
               _timed(lambda: dist.reduce_scatter_tensor(piece, plain), args.iters), 0.0, (ws - 1) / ws * n * 2)
        report("all_gather 256 MiB (kernel vs NCCL)", _timed(lambda: all_gather_(buf, ctrl), args.iters),
               _timed(lambda: dist.all_gather_into_tensor(plain, piece), args.iters), 0.0, (ws - 1) / ws * n * 2)
        report("broadcast 256 MiB (kernel vs NCCL)", _timed(lambda: broadcast_(buf, ctrl, root=0), args.iters),
               _timed(lambda: dist.broadcast(plain, src=0), args.iters), 0.0, n * 2)
        del buf, plain, piece

    # ---- full shard, one decoder block: gather of the ranks' pieces by the copy engine out of symmetric
    # memory (no kernel, no handshake) against an NCCL all-gather; reduce-scatter of the gradient images
    # with the accumulation into the owned piece and the clearing of the image in the same kernel against
    # NCCL reduce-scatter + add + memset
    if "unit" in groups:
        import ctypes

        from ..ops._lib import check as _check, lib as _lib_, ptr as _ptr

        U = args.unit_numel // (8 * ws) * (8 * ws)
        per = U // ws
        pieces = SymmetricBuffer(per, torch.bfloat16, dev)
        pieces.tensor.normal_(generator=gen)
        image = torch.empty(U, dtype=torch.bfloat16, device=dev)
        gimage = SymmetricBuffer(U, torch.bfloat16, dev)
        gplain = torch.empty(U, dtype=torch.bfloat16, device=dev)
        acc, tmp = torch.zeros(per, dtype=torch.bfloat16, device=dev), torch.empty(per, dtype=torch.bfloat16, device=dev)
        uctrl = PeerControl(dev)
        torch.cuda.synchronize()
        dist.barrier()

        def unit_gather():
            st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
            for k in range(ws):
                r = (rank + k) % ws
                _check(_lib_().kb_copy_async(ctypes.c_void_p(image.data_ptr() + r * per * 2),
                                             ctypes.c_void_p(pieces.peer_ptrs[r]), per * 2, st), "copy_async")

        def unit_reduce():
            mc = ctypes.c_void_p(gimage.multicast_ptr) if gimage.multicast_ptr else None
            _check(_lib_().kb_unit_reduce_bf16(gimage.ptrs, uctrl.flags.ptrs, mc, rank, ws, U, 1.0 / ws, _ptr(acc), 1,
                                               uctrl.next_epoch(2), 0, 256,
                                               ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)), "unit_reduce")

        def unit_reduce_lib():
            dist.reduce_scatter_tensor(tmp, gplain)
            acc.add_(tmp, alpha=1.0 / ws)
            gplain.zero_()

        report(f"full-shard unit gather, {U * 2 / 2 ** 20:.0f} MiB (copy engine vs NCCL all_gather)",
               _timed(unit_gather, args.iters), _timed(lambda: dist.all_gather_into_tensor(gplain, tmp), args.iters),
               0.0, (ws - 1) / ws * U * 2)
        report(f"full-shard unit reduce-scatter + accumulate + clear, {U * 2 / 2 ** 20:.0f} MiB (kernel vs NCCL + add + memset)",
               _timed(unit_reduce, args.iters), _timed(unit_reduce_lib, args.iters), 0.0, (ws - 1) / ws * U * 2)
        del pieces, image, gimage, gplain, acc, tmp

    if "optimizer" in groups:
        # ---- the data-parallel optimizer step on a buffer of the 1B model's size (1.15 G parameters): gradient
        # reduce-scatter + global clip + sharded AdamW + parameter all-gather, as one monolithic call and in
        # 25 MB buckets, against NCCL all-reduce + this package's single-GPU AdamW kernel on the whole vector
        from ..parallel.comm import GradReducer
        from ..trainer.optim import FusedAdamW
        from ..utils.flat_params import FlatParameters

        n_model = args.model_params // (8 * ws) * (8 * ws)

        class _One(torch.nn.Module):
            def __init__(self):
                super().__init__()
                self.w = torch.nn.Parameter(torch.zeros(n_model, dtype=torch.bfloat16, device=dev))

        link = 2 * (ws - 1) / ws * n_model * 2
        for label, cap in (("one launch", None), ("25 MB buckets", 25)):
            mod = _One()
            flat = FlatParameters(mod, with_grad=True, pad_to=8 * ws)
            red = GradReducer.create(flat, bucket_cap_mb=cap, overlap=cap is not None)
            opt = FusedAdamW(mod.parameters(), lr=1e-4, betas=(0.9, 0.95), weight_decay=0.01)
            opt.attach_flat(flat, allocate=False)
            opt.attach_reducer(red)
            flat.grad.normal_(generator=gen)

            def fused_step():
                opt.fused_clip(1.0)
                opt.step()

            fused_ms = _timed(fused_step, max(3, args.iters // 4))
            if cap is None:
                m = torch.zeros(n_model, dtype=torch.float32, device=dev)
                v = torch.zeros_like(m)
                g2 = flat.grad.clone()
                lr_step = torch.tensor([1e-4, 1.0], device=dev)
                sq = torch.zeros(1, device=dev)
                from ..ops._lib import check as _check, lib as _lib_, ptr as _ptr, stream as _stream

                def lib_step():
                    dist.all_reduce(g2)
                    sq.zero_()
                    _check(_lib_().kb_sumsq_bf16(_ptr(g2), n_model, _ptr(sq), _stream()), "sumsq")
                    _check(_lib_().kb_adamw_bf16(_ptr(flat.data), _ptr(g2), _ptr(m), _ptr(v), n_model, _ptr(lr_step), 0.9, 0.95,
                                                 1e-8, 0.01, 1.0 / ws, _ptr(sq), 1.0, _stream()), "adamw")

                base_ms = _timed(lib_step, max(3, args.iters // 4))
                del m, v, g2
            report(f"reduce+clip+AdamW+all_gather, {n_model / 1e9:.2f} G params ({label})", fused_ms, base_ms, 0.0, link)
            del mod, flat, red, opt
            torch.cuda.empty_cache()

    torch.cuda.synchronize()
    raise_on_device_error()
    if rank == 0:
        print(json.dumps({"world_size": ws, "tokens": T, "nvls": bool(args.nvls), "results": results}))
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
