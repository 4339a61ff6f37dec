"""Multi-GPU tests (2 ranks, one process per GPU): in-kernel NVLink collectives against NCCL,
the fused data-parallel optimizer step against a single-GPU run, and the bounded peer wait.
Every case runs on plain peer loads/stores with no multicast object bound (what the
fault-handling tests require); the collective and data-parallel parity cases run a second time
through the NVSwitch multicast (multimem) data plane, which is what a default run uses."""
import os

import pytest
import torch
import torch.distributed as dist

pytestmark = pytest.mark.gpu

if torch.cuda.device_count() < 2:
    pytest.skip("needs 2 GPUs", allow_module_level=True)

from khaosz_b200.parallel import ExecutorFactory, spawn_parallel_fn  # noqa: E402


_NVLS_OFF = {"KHAOSZ_B200_NVLS": "0", "NCCL_NVLS_ENABLE": "0", "TORCH_SYMM_MEM_DISABLE_MULTICAST": "1"}


def _spawn(fn, port, nvls=False, **kw):
    """Run ``fn`` on two ranks.  ``nvls=False``: no multicast object is created at all (not by
    this package, not by torch's symmetric memory, not by NCCL), so a rank that ends early never
    holds a multicast binding.  ``nvls=True``: the default data plane (multimem where available)."""
    saved = {k: os.environ.get(k) for k in _NVLS_OFF}
    for k, v in _NVLS_OFF.items():
        if nvls:
            os.environ.pop(k, None)
        else:
            os.environ[k] = v
    os.environ["KHAOSZ_B200_PG_TIMEOUT_S"] = "90"  # a failing rank must not keep the others waiting
    try:
        spawn_parallel_fn(fn, world_size=2, backend="nccl", master_addr="127.0.0.1", master_port=str(port), **kw)
    finally:
        for k, v in saved.items():
            if v is None:
                os.environ.pop(k, None)
            else:
                os.environ[k] = v


def _allreduce_case(expect_multicast=False):
    from khaosz_b200.ops import raise_on_device_error
    from khaosz_b200.parallel.comm import PeerControl, SymmetricBuffer, allreduce_

    rank = dist.get_rank()
    dev = torch.device("cuda", rank)
    n = 8 * 1000 * 1000 + 64
    buf = SymmetricBuffer(n, torch.bfloat16, dev)
    if not expect_multicast:
        assert buf.multicast_ptr == 0
    elif not buf.multicast_ptr:
        print("no multicast support on this box: the multimem path did not run")
    ctrl = PeerControl(dev)
    g = torch.Generator(device=dev).manual_seed(rank)
    src = torch.randn(n, device=dev, generator=g).to(torch.bfloat16)
    for it in range(3):
        buf.tensor.copy_(src)
        ref = src.float().clone()
        dist.all_reduce(ref)
        torch.cuda.synchronize()
        dist.barrier()
        allreduce_(buf, ctrl, scale=0.5)
        torch.cuda.synchronize()
        raise_on_device_error()
        err = (buf.tensor.float() - ref * 0.5).abs().max().item()
        assert err <= 2e-2 * ref.abs().max().item(), err
        dist.barrier()
    # timing, max over ranks
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    dist.barrier()
    e0.record()
    for _ in range(10):
        allreduce_(buf, ctrl, scale=1.0)
    e1.record()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) / 10], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    if rank == 0:
        print(f"kernel all-reduce {n * 2 / 1e6:.0f} MB, 2 ranks: {t.item():.3f} ms (bus {n * 2 / t.item() / 1e6:.0f} GB/s)")


@pytest.mark.parametrize("nvls,port", [(False, 29701), (True, 29711)])
def test_kernel_allreduce_matches_nccl(nvls, port):
    _spawn(_allreduce_case, port, nvls=nvls, expect_multicast=nvls)


def _collectives_case(expect_multicast=False):
    """Stand-alone reduce-scatter, all-gather and broadcast kernels against plain tensor arithmetic."""
    from khaosz_b200.ops import raise_on_device_error
    from khaosz_b200.parallel.comm import PeerControl, SymmetricBuffer, all_gather_, broadcast_, reduce_scatter

    rank, ws = dist.get_rank(), dist.get_world_size()
    dev = torch.device("cuda", rank)
    n = 16 * ws * 4099
    buf = SymmetricBuffer(n, torch.bfloat16, dev)
    assert bool(buf.multicast_ptr) == bool(expect_multicast and buf.multicast_ptr)
    ctrl = PeerControl(dev)
    srcs = [torch.randn(n, device=dev, generator=torch.Generator(device=dev).manual_seed(100 + r)).to(torch.bfloat16)
            for r in range(ws)]
    per = n // ws
    for it in range(2):
        # reduce-scatter (mean): my piece of the sum
        buf.tensor.copy_(srcs[rank])
        torch.cuda.synchronize(); dist.barrier()
        out = reduce_scatter(buf, ctrl, scale=1.0 / ws)
        torch.cuda.synchronize()
        want = sum(s_[rank * per:(rank + 1) * per].float() for s_ in srcs) / ws
        assert (out.float() - want).abs().max().item() <= 2e-2 * want.abs().max().item()
        assert torch.equal(buf.tensor, srcs[rank])            # the inputs are left alone
        dist.barrier()
        # all-gather: everybody ends with piece r of rank r
        buf.tensor.zero_()
        buf.tensor[rank * per:(rank + 1) * per].copy_(srcs[rank][rank * per:(rank + 1) * per])
        torch.cuda.synchronize(); dist.barrier()
        all_gather_(buf, ctrl)
        torch.cuda.synchronize()
        for r in range(ws):
            assert torch.equal(buf.tensor[r * per:(r + 1) * per], srcs[r][r * per:(r + 1) * per]), (it, r)
        dist.barrier()
        # broadcast from the last rank
        buf.tensor.copy_(srcs[rank])
        torch.cuda.synchronize(); dist.barrier()
        broadcast_(buf, ctrl, root=ws - 1)
        torch.cuda.synchronize()
        assert torch.equal(buf.tensor, srcs[ws - 1])
        dist.barrier()
    raise_on_device_error()


@pytest.mark.parametrize("nvls,port", [(False, 29715), (True, 29716)])
def test_kernel_reduce_scatter_all_gather_broadcast(nvls, port):
    _spawn(_collectives_case, port, nvls=nvls, expect_multicast=nvls)


def _timeout_case():
    from khaosz_b200.ops import _lib
    from khaosz_b200.parallel.comm import PeerControl

    rank = dist.get_rank()
    dev = torch.device("cuda", rank)
    ctrl = PeerControl(dev)
    ctrl.barrier()
    torch.cuda.synchronize()
    assert _lib.lib().kb_last_error() == 0
    dist.barrier()
    if rank == 0:
        # a barrier nobody else joins (a flag that nothing sets): must give up after ~200 ms
        ctrl.barrier(budget_ms=200, slot=3)
        torch.cuda.synchronize()
        assert _lib.lib().kb_last_error() == 5  # KB_ERR_TIMEOUT_PEER
    dist.barrier()  # host-side: rank 1 learns nothing was lost
    if rank == 1:
        ctrl.next_epoch()  # keep the epoch counters of both ranks in step
    ctrl.barrier()  # the context and the control buffer are still usable
    torch.cuda.synchronize()
    assert _lib.lib().kb_last_error() == 0
    x = torch.ones(4, device=dev)
    dist.all_reduce(x)
    assert x.sum().item() == 8


def test_peer_wait_is_bounded_and_context_survives():
    _spawn(_timeout_case, 29702)


def _cfg(layers=2):
    from khaosz_b200 import AutoRegressiveLMConfig

    return AutoRegressiveLMConfig(vocab_size=4096, dim=512, n_layers=layers, norm_eps=1e-5, dim_ffn=1408, tie_weight=True,
                                  max_len=256, rope_theta=1e4, n_heads=4, n_kv_heads=2)


def _train(mode, world, rank, device, steps=4, accum=2, cuda_graph=False, overlap=False, layers=2):
    from khaosz_b200 import AutoRegressiveLM
    from khaosz_b200.trainer import FusedAdamW, StrategyFactory

    torch.manual_seed(3407)
    model = AutoRegressiveLM(_cfg(layers)).to(device=device, dtype=torch.bfloat16)
    # ~1 MB buckets handed over during the backward pass: several per step on this small model
    extra = {"bucket_cap_mb": 1, "overlap_grad_reduce": True} if overlap else {}
    ex = ExecutorFactory.create(mode, grad_accum_steps=accum, cuda_graph=cuda_graph, **extra)
    opt = FusedAdamW(model.parameters(), lr=1e-3, betas=(0.9, 0.95), weight_decay=0.01)
    model, opt, _, _ = ex.prepare(model, opt, None, None)
    strat = StrategyFactory.create("seq", model, device, label_smoothing=0.05)
    g = torch.Generator().manual_seed(11)
    data = torch.randint(0, 4096, (steps * accum, 2 * world, 129), generator=g)
    losses = []
    for i in range(steps * accum):
        mine = (data[i] if mode == "tp" else data[i, 2 * rank:2 * rank + 2]).to(device)
        with ex.accumulate(model):
            loss = ex.micro_step(strat, {"input_ids": mine[:, :-1].contiguous(), "target_ids": mine[:, 1:].contiguous()})
            if ex.sync_gradients:
                opt.fused_clip(1.0)
                opt.step()
                opt.zero_grad()
        losses.append(loss.detach().float())
    if cuda_graph:
        assert ex._graphed is not None and not ex._graphed.disabled and any("graph" in e for e in ex._graphed.entries.values()), \
            "the micro-step was not captured"
    return torch.stack(losses), model, ex, opt


def _dp_case(mode, out, overlap=False):
    from khaosz_b200.ops import raise_on_device_error

    rank = dist.get_rank()
    dev = torch.device("cuda", rank)
    losses, model, ex, opt = _train(mode, 2, rank, dev, overlap=overlap)
    dist.all_reduce(losses)
    losses /= 2
    raise_on_device_error()
    assert ex._reducer is not None and ex._fused, "the fused NVLink kernel path was not taken"
    sd = ex.unwrap_model(model)
    osd = opt.state_dict()  # gathers the sharded moments (collective)
    # both ranks must hold identical parameters after the in-kernel all-gather
    flat = ex.flat.data.float()
    other = flat.clone()
    dist.broadcast(other, src=0)
    assert torch.equal(flat, other)
    if rank == 0:
        torch.save({"losses": losses.cpu(), "sd": {k: v.cpu() for k, v in sd.items()},
                    "m0": osd["state"][0]["exp_avg"]}, out)


def _block_case(out):
    """Block-granular full shard: five blocks through two weight images, gathered and reduced on a side stream."""
    from khaosz_b200.ops import raise_on_device_error

    rank = dist.get_rank()
    dev = torch.device("cuda", rank)
    losses, model, ex, opt = _train("fsdp_block", 2, rank, dev, layers=5)
    dist.all_reduce(losses)
    losses /= 2
    raise_on_device_error()
    u = ex.units
    assert u._sym and u.gathers > 0 and u.reductions == 4 * 2 * 5, "the side-stream collectives did not run"
    assert u.data.numel() == sum(x.numel for x in u.units) // 2 + u.rest_numel
    sd = ex.unwrap_model(model)
    osd = opt.state_dict()
    if rank == 0:
        torch.save({"losses": losses.cpu(), "sd": {k: v.cpu() for k, v in sd.items()},
                    "m0": osd["state"][0]["exp_avg"]}, out)


def _tp_train_case(out, mode="tp", cuda_graph=False):
    from khaosz_b200.ops import raise_on_device_error
    from khaosz_b200.parallel.tensor_parallel import TPContext

    rank = dist.get_rank()
    dev = torch.device("cuda", rank)
    if cuda_graph:  # a stuck rank reports where it is; the kernels' bounded waits and the error word end the run
        import faulthandler

        faulthandler.dump_traceback_later(60, exit=False)
    losses, model, ex, opt = _train(mode, 2, rank, dev, cuda_graph=cuda_graph)
    if cuda_graph:
        faulthandler.cancel_dump_traceback_later()
    dist.all_reduce(losses)
    losses /= 2
    raise_on_device_error()
    assert TPContext.get().use_kernels, "the fused tensor-parallel kernels were not used"
    sd = ex.unwrap_model(model)
    if rank == 0:
        torch.save({"losses": losses.cpu(), "sd": {k: v.cpu() for k, v in sd.items()}}, out)


@pytest.mark.parametrize("mode,port", [("ddp", 29703), ("fsdp_zero1", 29704), ("tp", 29707), ("fsdp_full", 29708),
                                       ("tp_graph", 29709), ("ddp_nvls", 29712), ("fsdp_zero1_nvls", 29713),
                                       ("ddp_overlap", 29714), ("fsdp_block", 29715), ("fsdp_block_nvls", 29716)])
def test_fused_data_parallel_step_matches_single_gpu(mode, port, tmp_path):
    out = str(tmp_path / "dp.pt")
    nvls = mode.endswith("_nvls")
    overlap = mode.endswith("_overlap")
    mode = mode.split("_nvls")[0].split("_overlap")[0]
    layers = 2
    if mode == "fsdp_block":
        layers = 5
        _spawn(_block_case, port, nvls=nvls, out=out)
    elif mode == "tp_graph":   # forward+backward of the tensor-parallel micro-step replayed as a CUDA graph
        _spawn(_tp_train_case, port, out=out, mode="tp", cuda_graph=True)
    elif mode in ("tp", "fsdp_full"):
        _spawn(_tp_train_case, port, out=out, mode=mode)
    else:
        _spawn(_dp_case, port, nvls=nvls, mode=mode, out=out, overlap=overlap)
    got = torch.load(out)
    # single GPU over the global batch
    from khaosz_b200 import AutoRegressiveLM
    from khaosz_b200.trainer import FusedAdamW, StrategyFactory

    torch.manual_seed(3407)
    dev = torch.device("cuda", 0)
    model = AutoRegressiveLM(_cfg(layers)).to(device=dev, dtype=torch.bfloat16)
    init = {k: v.detach().float().cpu().clone() for k, v in model.state_dict().items()}
    ex = ExecutorFactory.create("none", grad_accum_steps=2)
    opt = FusedAdamW(model.parameters(), lr=1e-3, betas=(0.9, 0.95), weight_decay=0.01)
    model, opt, _, _ = ex.prepare(model, opt, None, None)
    strat = StrategyFactory.create("seq", model, dev, label_smoothing=0.05)
    g = torch.Generator().manual_seed(11)
    data = torch.randint(0, 4096, (8, 4, 129), generator=g)
    losses = []
    for i in range(8):
        b = data[i].to(dev)
        with ex.accumulate(model):
            loss = strat({"input_ids": b[:, :-1], "target_ids": b[:, 1:]})
            ex.backward(loss / 2)
            if ex.sync_gradients:
                opt.fused_clip(1.0)
                opt.step()
                opt.zero_grad()
        losses.append(loss.item())
    ref = torch.tensor(losses)
    assert torch.allclose(got["losses"], ref, rtol=2e-2, atol=2e-2), (got["losses"], ref)
    sd = model.state_dict()
    worst = max((got["sd"][k].float() - v.float().cpu()).abs().max().item() for k, v in sd.items())
    assert worst < 2e-2, worst
    # the *updates* must agree, not only the weights: four AdamW steps at lr 1e-3 move a weight by a
    # few 1e-3, so a rank that never applied an update would pass the absolute check above
    moved = 0
    for k, v in sd.items():
        d_ref = v.float().cpu() - init[k]
        d_got = got["sd"][k].float() - init[k]
        if d_ref.abs().max().item() < 5e-4:
            # bf16 weights without an fp32 master cannot follow every update (a norm weight at 1.0 needs a
            # step of 2^-9 to move at all): then the parallel run must not have moved either
            assert d_got.abs().max().item() < 8e-3, k
            continue
        moved += 1
        cos = torch.nn.functional.cosine_similarity(d_ref.flatten(), d_got.flatten(), dim=0).item()
        assert cos > 0.9, f"{k}: update direction differs from the single-GPU run (cosine {cos:.3f})"
        ratio = d_got.norm().item() / d_ref.norm().item()
        assert 0.8 < ratio < 1.25, f"{k}: update size differs from the single-GPU run (ratio {ratio:.3f})"
    assert moved >= len(sd) // 2, f"only {moved} of {len(sd)} tensors moved in the single-GPU run"
    if "m0" in got:
        assert got["m0"].shape == sd["embed_tokens.weight"].shape


def _tp_kernels_case():
    from khaosz_b200.ops import raise_on_device_error
    from khaosz_b200.parallel.tensor_parallel import TPContext, _comm_gemm

    rank, ws = dist.get_rank(), dist.get_world_size()
    dev = torch.device("cuda", rank)
    tp = TPContext.get()
    assert tp.use_kernels
    g = torch.Generator(device=dev).manual_seed(100 + rank)
    M, K, N = 512, 640, 768  # M = tokens over all ranks
    x_shard = torch.randn(M // ws, K, device=dev, generator=g).to(torch.bfloat16)
    w = (torch.randn(N, K, device=dev, generator=g) * 0.1).to(torch.bfloat16)

    def gather(t):
        parts = [torch.empty_like(t) for _ in range(ws)]
        dist.all_gather(parts, t)
        return torch.cat(parts, 0)

    def close(got, ref):
        err = (got.float() - ref).abs().max().item()
        assert err <= 2e-2 * ref.abs().max().item() + 2e-2, err

    x_full = gather(x_shard).float()
    for _ in range(2):  # twice: buffers, epochs and the grid barrier are reused
        # all-gather -> GEMM (K-major gathered A)
        close(_comm_gemm(tp, x_shard, w, a_gather=True, tag="t1"), x_full @ w.float().t())
        # gathered weights (FSDP style): B rows sharded over ranks
        w_shard = w[rank * (N // ws):(rank + 1) * (N // ws)].contiguous() if (N // ws) % 256 == 0 else None
        # GEMM -> reduce-scatter and GEMM -> all-reduce
        xa = torch.randn(M, K, device=dev, generator=g).to(torch.bfloat16)
        total = xa.float() @ w.float().t()
        dist.all_reduce(total)
        rs = _comm_gemm(tp, xa, w, c_mode=1, tag="t2")
        close(rs, total[rank * (M // ws):(rank + 1) * (M // ws)])
        ar = _comm_gemm(tp, xa[:24].contiguous(), w, c_mode=2, tag="t3")
        close(ar, total[:24])
        # MN-major gathered operand: dW = dy^T all_gather(x)   (reduction dimension sharded)
        dy = torch.randn(M, N, device=dev, generator=g).to(torch.bfloat16)
        dw = _comm_gemm(tp, dy, x_shard, a_mn=True, b_mn=True, b_gather=True, tag="t4")
        close(dw, dy.float().t() @ x_full)
        torch.cuda.synchronize()
        raise_on_device_error()
    # weights sharded by rows and gathered inside the GEMM (the FSDP use of the same kernel)
    N2 = 256 * ws
    w2 = (torch.randn(N2 // ws, K, device=dev, generator=g) * 0.1).to(torch.bfloat16)
    y = _comm_gemm(tp, xa, w2, b_gather=True, tag="t5")
    close(y, xa.float() @ gather(w2).float().t())
    # shards that are not whole 128-row chunks take the direct path (tiles read from the owner)
    xs = torch.randn(192, K, device=dev, generator=g).to(torch.bfloat16)
    dy2 = torch.randn(192 * ws, N, device=dev, generator=g).to(torch.bfloat16)
    dw2 = _comm_gemm(tp, dy2, xs, a_mn=True, b_mn=True, b_gather=True, tag="t6")
    close(dw2, dy2.float().t() @ gather(xs).float())
    torch.cuda.synchronize()
    raise_on_device_error()


def test_fused_comm_gemm_kernels():
    _spawn(_tp_kernels_case, 29705)


def _tp_mlp_case(out):
    """Column-parallel -> SwiGLU -> row-parallel MLP on sequence-sharded tokens, forward and
    backward through the fused kernels, against the same MLP on one GPU."""
    from khaosz_b200 import ops
    from khaosz_b200.parallel.tensor_parallel import ColumnParallelLinear, RowParallelLinear

    rank, ws = dist.get_rank(), dist.get_world_size()
    dev = torch.device("cuda", rank)
    torch.manual_seed(7)
    T, D, Fh = 512, 512, 1024
    x_full = torch.randn(T, D, device=dev).to(torch.bfloat16)
    wg = (torch.randn(Fh, D, device=dev) * 0.05).to(torch.bfloat16)
    wu = (torch.randn(Fh, D, device=dev) * 0.05).to(torch.bfloat16)
    wd = (torch.randn(D, Fh, device=dev) * 0.05).to(torch.bfloat16)
    go_full = torch.randn(T, D, device=dev).to(torch.bfloat16)
    gate_up = ColumnParallelLinear(D, 2 * Fh).to(dev, torch.bfloat16)
    down = RowParallelLinear(Fh, D).to(dev, torch.bfloat16)
    n = Fh // ws
    with torch.no_grad():  # local slices: [gate_r | up_r]
        gate_up.weight.copy_(torch.cat([wg[rank * n:(rank + 1) * n], wu[rank * n:(rank + 1) * n]], 0))
    down.load_state_dict({"weight": wd})
    x = x_full[rank * (T // ws):(rank + 1) * (T // ws)].clone().requires_grad_()
    y = down(ops.swiglu(gate_up(x)))
    y.backward(go_full[rank * (T // ws):(rank + 1) * (T // ws)])
    ops.raise_on_device_error()
    # single-GPU oracle in fp32
    xf = x_full.float().requires_grad_()
    wgf, wuf, wdf = (t.float().requires_grad_() for t in (wg, wu, wd))
    ref = ((xf @ wuf.t()) * torch.nn.functional.silu(xf @ wgf.t())) @ wdf.t()
    ref.backward(go_full.float())
    sl = slice(rank * (T // ws), (rank + 1) * (T // ws))

    def close(got, want, name):
        err = (got.float() - want).abs().max().item()
        assert err <= 3e-2 * want.abs().max().item() + 3e-2, (name, err)

    close(y, ref[sl], "y")
    close(x.grad, xf.grad[sl], "dx")
    close(gate_up.weight.grad[:n], wgf.grad[rank * n:(rank + 1) * n], "dwg")
    close(gate_up.weight.grad[n:], wuf.grad[rank * n:(rank + 1) * n], "dwu")
    close(down.weight.grad, wdf.grad[:, rank * n:(rank + 1) * n], "dwd")
    if rank == 0:
        open(out, "w").write("ok")


def test_tensor_parallel_mlp_matches_single_gpu(tmp_path):
    out = str(tmp_path / "tp.txt")
    _spawn(_tp_mlp_case, 29706, out=out)
    assert open(out).read() == "ok"


# ---- tensor-parallel serving: rank 0 drives the engine, rank 1 replays the announced steps ----
class _Ids:
    stop_ids: list = []

    def encode(self, text, **_):
        return list(text) if not isinstance(text, str) else [int(t) for t in text.split()]

    def decode(self, ids, **_):
        return " ".join(str(i) for i in ids) + " "


def _tp_infer_case(out):
    from khaosz_b200 import AutoRegressiveLM
    from khaosz_b200.inference import InferenceEngine
    from khaosz_b200.inference.tp import TPInferenceLM, serve_worker
    from khaosz_b200.ops import raise_on_device_error

    rank = dist.get_rank()
    dev = torch.device("cuda", rank)
    torch.manual_seed(3407)
    dense = AutoRegressiveLM(_cfg()).to(device=dev, dtype=torch.bfloat16).eval()
    tp = TPInferenceLM(dense).eval()
    ids = torch.randint(0, 4096, (2, 64), generator=torch.Generator().manual_seed(2)).to(dev)
    with torch.inference_mode():
        ref = dense(ids)["logits"].float()
        got = tp(ids)["logits"].float()
    err = (got - ref).abs().max().item() / ref.abs().max().item()
    assert err < 3e-2, err
    tok = _Ids()
    if rank != 0:
        serve_worker(tp, tok, max_batch_size=4, max_seq_len=160, page_size=16)
    else:
        g = torch.Generator().manual_seed(5)
        prompts = [torch.randint(0, 4096, (n,), generator=g).tolist() for n in (40, 17, 90)]
        with InferenceEngine(tp, tok, max_batch_size=4, max_seq_len=160, page_size=16) as eng:
            texts = eng.generate(prompts, max_tokens=12, temperature=1.0, top_k=1, top_p=1.0)
            graphs = sum(1 for s in eng.scheduler._executor._slots.values() if s.graph is not None)
        toks = [[int(t) for t in text.split()] for text in texts]
        assert all(len(t) == 12 and all(0 <= x < 4096 for x in t) for t in toks), toks
        # the first generated token comes from the prefill logits: it must be the dense model's arg-max
        with torch.inference_mode():
            first = [int(dense(torch.tensor([p], device=dev))["logits"][0, -1].float().argmax()) for p in prompts]
        torch.save({"first_got": [t[0] for t in toks], "first_want": first, "graphs": graphs}, out)
    torch.cuda.synchronize()
    raise_on_device_error()


def test_tensor_parallel_serving(tmp_path):
    out = str(tmp_path / "tp_inf.pt")
    _spawn(_tp_infer_case, 29710, out=out)
    r = torch.load(out)
    assert sum(a == b for a, b in zip(r["first_got"], r["first_want"])) >= 2, r   # bf16 ties may flip one
    assert r["graphs"] >= 1, "the tensor-parallel decode step was not replayed as a CUDA graph"
