"""Multi-GPU tests (2 ranks, one process per GPU): in-kernel NVLink collectives against NCCL,
the fused data-parallel optimizer step against a single-GPU run, and the bounded peer wait.
Plain peer loads/stores only (multicast off), as required for fault-handling tests."""
import os

import pytest
import torch
import torch.distributed as dist

pytestmark = pytest.mark.gpu

if torch.cuda.device_count() < 2:
    pytest.skip("needs 2 GPUs", allow_module_level=True)

from khaosz_b200.parallel import ExecutorFactory, spawn_parallel_fn  # noqa: E402


def _spawn(fn, port, **kw):
    os.environ["KHAOSZ_B200_NVLS"] = "0"
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    spawn_parallel_fn(fn, world_size=2, backend="nccl", master_addr="127.0.0.1", master_port=str(port), **kw)


def _allreduce_case():
    from khaosz_b200.ops import raise_on_device_error
    from khaosz_b200.parallel.comm import PeerControl, SymmetricBuffer, allreduce_

    rank = dist.get_rank()
    dev = torch.device("cuda", rank)
    n = 8 * 1000 * 1000 + 64
    buf = SymmetricBuffer(n, torch.bfloat16, dev)
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


def test_kernel_allreduce_matches_nccl():
    _spawn(_allreduce_case, 29701)


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


def _cfg():
    from khaosz_b200 import AutoRegressiveLMConfig

    return AutoRegressiveLMConfig(vocab_size=4096, dim=512, n_layers=2, norm_eps=1e-5, dim_ffn=1408, tie_weight=True,
                                  max_len=256, rope_theta=1e4, n_heads=4, n_kv_heads=2)


def _train(mode, world, rank, device, steps=4, accum=2):
    from khaosz_b200 import AutoRegressiveLM
    from khaosz_b200.trainer import FusedAdamW, StrategyFactory

    torch.manual_seed(3407)
    model = AutoRegressiveLM(_cfg()).to(device=device, dtype=torch.bfloat16)
    ex = ExecutorFactory.create(mode, grad_accum_steps=accum)
    opt = FusedAdamW(model.parameters(), lr=1e-3, betas=(0.9, 0.95), weight_decay=0.01)
    model, opt, _, _ = ex.prepare(model, opt, None, None)
    strat = StrategyFactory.create("seq", model, device, label_smoothing=0.05)
    g = torch.Generator().manual_seed(11)
    data = torch.randint(0, 4096, (steps * accum, 2 * world, 129), generator=g)
    losses = []
    for i in range(steps * accum):
        mine = data[i, 2 * rank:2 * rank + 2].to(device)
        with ex.accumulate(model):
            loss = strat({"input_ids": mine[:, :-1], "target_ids": mine[:, 1:]})
            ex.backward(loss / accum)
            if ex.sync_gradients:
                opt.fused_clip(1.0)
                opt.step()
                opt.zero_grad()
        losses.append(loss.detach().float())
    return torch.stack(losses), model, ex, opt


def _dp_case(mode, out):
    from khaosz_b200.ops import raise_on_device_error

    rank = dist.get_rank()
    dev = torch.device("cuda", rank)
    losses, model, ex, opt = _train(mode, 2, rank, dev)
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


@pytest.mark.parametrize("mode,port", [("ddp", 29703), ("fsdp", 29704)])
def test_fused_data_parallel_step_matches_single_gpu(mode, port, tmp_path):
    out = str(tmp_path / "dp.pt")
    _spawn(_dp_case, port, mode=mode, out=out)
    got = torch.load(out)
    # single GPU over the global batch
    from khaosz_b200 import AutoRegressiveLM
    from khaosz_b200.trainer import FusedAdamW, StrategyFactory

    torch.manual_seed(3407)
    dev = torch.device("cuda", 0)
    model = AutoRegressiveLM(_cfg()).to(device=dev, dtype=torch.bfloat16)
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
    assert got["m0"].shape == sd["embed_tokens.weight"].shape
