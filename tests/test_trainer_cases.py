"""Case-by-case behaviour of the schedulers, the gradient-checkpointing callback, trainer runs with
different batch settings and the launch helpers (the behaviours the reference pins in
``tests/trainer/*.py`` and ``tests/parallel/test_parallel.py``)."""
import json
import math
import os
import random

import pytest
import torch
import torch.distributed as dist

from conftest import RandomTokens, tiny_config
from khaosz_b200 import AutoRegressiveLM, TrainConfig
from khaosz_b200.models.components.block import DecoderBlock
from khaosz_b200.parallel import spawn_parallel_fn
from khaosz_b200.parallel.setup import only_on_rank
from khaosz_b200.trainer import (CallbackFactory, FusedAdamW, GradientCheckpointingCallback, SchedulerFactory, Trainer)


def _opt(lr=1.0, groups=1):
    return torch.optim.SGD([{"params": [torch.nn.Parameter(torch.zeros(1))], "lr": lr * (i + 1)} for i in range(groups)], lr=lr)


def _curve(opt, sched, steps):
    lrs = [opt.param_groups[0]["lr"]]
    for _ in range(steps):
        opt.step()
        sched.step()
        lrs.append(opt.param_groups[0]["lr"])
    return lrs


# ---- schedulers -------------------------------------------------------------------------------
def test_cosine_schedule_matches_its_formula_for_random_settings():
    rng = random.Random(0)
    for _ in range(20):
        warmup, decay = rng.randint(1, 20), rng.randint(1, 50)
        min_rate, base = rng.choice([0.0, 0.05, 0.3]), rng.choice([1.0, 3e-4])
        opt = _opt(base)
        lrs = _curve(opt, SchedulerFactory.create(opt, "cosine", warmup_steps=warmup, lr_decay_steps=decay, min_rate=min_rate),
                     warmup + decay + 5)
        for step, lr in enumerate(lrs):
            if step < warmup:
                want = max(min_rate, step / warmup)
            else:
                want = max(min_rate, 0.5 * (1 + math.cos(math.pi * min((step - warmup) / decay, 1.0))))
            assert lr == pytest.approx(base * want, rel=1e-9, abs=1e-15), (warmup, decay, min_rate, step)


def test_cosine_schedule_first_and_last_rates():
    opt = _opt(2.0)
    lrs = _curve(opt, SchedulerFactory.create(opt, "cosine", warmup_steps=10, lr_decay_steps=20), 60)
    assert lrs[0] == pytest.approx(2.0 * 0.05)              # the first step already runs at min_rate, not zero
    assert max(lrs) == pytest.approx(2.0) and lrs[10] == pytest.approx(2.0)
    assert lrs[30] == pytest.approx(2.0 * 0.05) and lrs[60] == pytest.approx(2.0 * 0.05)   # held after the decay
    assert all(a >= b - 1e-12 for a, b in zip(lrs[10:], lrs[11:]))                          # monotone decay


def test_schedules_scale_every_parameter_group():
    opt = _opt(1.0, groups=2)
    sched = SchedulerFactory.create(opt, "cosine", warmup_steps=2, lr_decay_steps=4, min_rate=0.0)
    for _ in range(2):
        opt.step()
        sched.step()
    assert [g["lr"] for g in opt.param_groups] == pytest.approx([1.0, 2.0])


@pytest.mark.parametrize("kind,kwargs", [("cosine", dict(warmup_steps=1, lr_decay_steps=1)),
                                         ("cosine", dict(warmup_steps=3, lr_decay_steps=0)),
                                         ("sgdr", dict(warmup_steps=1, cycle_length=1)),
                                         ("sgdr", dict(warmup_steps=2, cycle_length=3, t_mult=1))])
def test_schedule_edge_settings_stay_finite(kind, kwargs):
    opt = _opt()
    lrs = _curve(opt, SchedulerFactory.create(opt, kind, **kwargs), 12)
    assert all(math.isfinite(lr) and 0.0 <= lr <= 1.0 + 1e-12 for lr in lrs)


def test_sgdr_restarts_with_growing_cycles():
    opt = _opt()
    lrs = _curve(opt, SchedulerFactory.create(opt, "sgdr", warmup_steps=2, cycle_length=4, min_rate=0.1, t_mult=2), 30)
    restarts = [i for i in range(3, 31) if lrs[i] == pytest.approx(1.0)]
    assert restarts == [6, 14, 30]                      # cycles of 4, 8 and 16 steps after the warm-up
    assert min(lrs[2:]) >= 0.1 - 1e-12 and lrs[5] < 0.3


def test_scheduler_state_survives_a_checkpoint():
    opt = _opt(0.5)
    sched = SchedulerFactory.create(opt, "sgdr", warmup_steps=3, cycle_length=5, min_rate=0.2, t_mult=3)
    _curve(opt, sched, 11)
    state = sched.state_dict()
    assert {"warmup_steps", "cycle_length", "min_rate", "t_mult", "last_epoch"} <= set(state)
    state = json.loads(json.dumps({k: v for k, v in state.items() if not callable(v)}, default=list))
    opt2 = _opt(0.5)
    other = SchedulerFactory.create(opt2, "sgdr", warmup_steps=1, cycle_length=1)
    other.load_state_dict(state)
    assert (other.warmup_steps, other.cycle_length, other.min_rate, other.t_mult, other.last_epoch) == (3, 5, 0.2, 3, 11)
    assert _curve(opt2, other, 6)[1:] == pytest.approx(_curve(opt, sched, 6)[1:])


def test_scheduler_registry():
    assert set(SchedulerFactory.available_types()) >= {"cosine", "sgdr"}
    with pytest.raises(ValueError, match="Unknown component"):
        SchedulerFactory.create(_opt(), "polynomial")
    with pytest.raises(TypeError):
        SchedulerFactory.register("bad")(dict)


# ---- gradient checkpointing ---------------------------------------------------------------------
def test_checkpointing_wraps_and_restores_the_listed_modules():
    model = AutoRegressiveLM(tiny_config())
    cb = GradientCheckpointingCallback([DecoderBlock])
    originals = [layer.forward for layer in model.layers]
    model.apply(cb._enable)
    assert all(hasattr(layer, "_original_forward") for layer in model.layers)
    assert not hasattr(model.norm, "_original_forward") and not hasattr(model, "_original_forward")
    model.apply(cb._enable)                             # enabling twice does not nest the wrappers
    assert all(layer._original_forward == orig for layer, orig in zip(model.layers, originals))
    model.apply(cb._disable)
    assert not any(hasattr(layer, "_original_forward") for layer in model.layers)
    assert all(layer.forward == orig for layer, orig in zip(model.layers, originals))


def test_checkpointing_without_modules_touches_nothing():
    model = AutoRegressiveLM(tiny_config())
    for cb in (GradientCheckpointingCallback(), GradientCheckpointingCallback([])):
        model.apply(cb._enable)
        assert not any(hasattr(m, "_original_forward") for m in model.modules())


def test_checkpointing_keeps_outputs_and_gradients():
    torch.manual_seed(0)
    model = AutoRegressiveLM(tiny_config())
    ids = torch.randint(0, 300, (2, 8))
    model(ids)["logits"].sum().backward()
    want_out = model(ids)["logits"].detach()
    want_grad = {n: p.grad.clone() for n, p in model.named_parameters()}
    model.zero_grad()
    model.apply(GradientCheckpointingCallback([DecoderBlock])._enable)
    out = model(ids)["logits"]
    assert torch.equal(out.detach(), want_out)
    out.sum().backward()
    for n, p in model.named_parameters():
        assert p.grad is not None and torch.allclose(p.grad, want_grad[n], atol=1e-6), n


def _config(tmp_path, **over):
    cfg = tiny_config()
    base = dict(model_fn=lambda: AutoRegressiveLM(cfg), strategy="seq", dataset=RandomTokens(n=24),
                optimizer_fn=lambda m: FusedAdamW(m.parameters(), lr=1e-3),
                scheduler_fn=lambda o: SchedulerFactory.create(o, "cosine", warmup_steps=2, lr_decay_steps=20),
                batch_per_device=4, ckpt_dir=str(tmp_path / "ck"), log_dir=str(tmp_path / "logs"), ckpt_interval=1000,
                log_interval=1, device_type="cpu", n_epoch=1)
    base.update(over)
    return TrainConfig(**base)


def _losses(tmp_path):
    logs = tmp_path / "logs"
    return [json.loads(line)["loss"] for f in sorted(os.listdir(logs)) for line in open(logs / f)]


def test_checkpointing_through_the_trainer_gives_the_same_losses(tmp_path):
    torch.manual_seed(0)                                # same initial weights for both runs
    Trainer(_config(tmp_path / "plain")).train()
    torch.manual_seed(0)
    Trainer(_config(tmp_path / "ckpt", gradient_checkpointing_modules=[DecoderBlock])).train()
    assert _losses(tmp_path / "ckpt") == pytest.approx(_losses(tmp_path / "plain"), rel=1e-5)


# ---- trainer runs -------------------------------------------------------------------------------
@pytest.mark.parametrize("batch", [1, 2, 8])
def test_trainer_runs_with_different_batch_sizes(tmp_path, batch):
    Trainer(_config(tmp_path, batch_per_device=batch)).train()
    losses = _losses(tmp_path)
    assert len(losses) == 24 // batch and all(math.isfinite(x) for x in losses)
    assert (tmp_path / "ck" / f"epoch_0_iter_{24 // batch}" / "model.safetensors").exists()


def test_accumulated_micro_batches_train_like_one_large_batch(tmp_path):
    sgd = lambda m: torch.optim.SGD(m.parameters(), lr=0.1)
    const = lambda o: torch.optim.lr_scheduler.LambdaLR(o, lambda _: 1.0)
    common = dict(optimizer_fn=sgd, scheduler_fn=const, max_grad_norm=0.0)
    torch.manual_seed(0)
    Trainer(_config(tmp_path / "big", batch_per_device=8, grad_accum_steps=1, **common)).train()
    torch.manual_seed(0)
    Trainer(_config(tmp_path / "acc", batch_per_device=2, grad_accum_steps=4, **common)).train()
    from khaosz_b200.serialization import Checkpoint

    big = Checkpoint.load(str(tmp_path / "big" / "ck" / "epoch_0_iter_3")).state_dict
    acc = Checkpoint.load(str(tmp_path / "acc" / "ck" / "epoch_0_iter_12")).state_dict
    for k, v in big.items():
        assert torch.allclose(acc[k], v, atol=1e-5), k


def test_accumulation_with_checkpointing_and_validation_together(tmp_path):
    cfg = _config(tmp_path, batch_per_device=2, grad_accum_steps=3, gradient_checkpointing_modules=[DecoderBlock],
                  val_split=0.25, val_step=1, metrics=["loss", "lr", "val_loss"])
    Trainer(cfg).train()
    rows = [json.loads(line) for f in sorted(os.listdir(tmp_path / "logs")) for line in open(tmp_path / "logs" / f)]
    assert rows and rows[-1]["val_loss"] > 0 and all(math.isfinite(r["loss"]) for r in rows)


def test_user_callbacks_run_after_the_default_ones(tmp_path):
    order = []

    class First:
        def on_train_begin(self, ctx):
            order.append(("first", type(ctx.optimizer).__name__))

        def on_optimizer_step(self, ctx):
            order.append(("step", ctx.iteration))

    class Second:
        def on_train_begin(self, ctx):
            order.append(("second", None))

        def on_train_end(self, ctx):
            order.append(("end", ctx.iteration))

    trainer = Trainer(_config(tmp_path, batch_per_device=8), callbacks=[First(), Second()])
    names = [type(cb).__name__ for cb in trainer.callbacks]
    assert names[-2:] == ["First", "Second"] and names[0] == "GradientCheckpointingCallback"
    trainer.train()
    assert order[0][0] == "first" and order[1] == ("second", None) and order[-1] == ("end", 3)
    assert [o for o in order if o[0] == "step"] == [("step", 1), ("step", 2), ("step", 3)]


def test_callback_registry():
    for name in ("gradient_clipping", "gradient_checkpointing", "checkpoint", "progress_bar", "metric_logger", "validation",
                 "device_health", "throughput"):
        assert CallbackFactory.is_registered(name), name
    with pytest.raises(ValueError, match="Unknown component"):
        CallbackFactory.create("no_such_callback")


def test_train_config_requires_its_core_fields():
    with pytest.raises(ValueError, match="model_fn is required"):
        TrainConfig(strategy="seq", dataset=[1], optimizer_fn=len, scheduler_fn=len)
    with pytest.raises(ValueError, match="dataset is required"):
        TrainConfig(model_fn=len, strategy="seq", optimizer_fn=len, scheduler_fn=len)
    cfg = TrainConfig(model_fn=len, strategy="seq", dataset=[1], optimizer_fn=len, scheduler_fn=len)
    assert (cfg.n_epoch, cfg.batch_per_device, cfg.grad_accum_steps, cfg.max_grad_norm) == (1, 4, 1, 1.0)
    assert (cfg.parallel_mode, cfg.nprocs, cfg.backend, cfg.random_seed) == ("none", 1, "nccl", 3407)


# ---- launch helpers -----------------------------------------------------------------------------
def _rank_files(out_dir):
    @only_on_rank(0, sync=True)
    def only_first():
        open(os.path.join(out_dir, "only_first"), "w").write(str(dist.get_rank()))
        return "done"

    result = only_first()
    assert result == ("done" if dist.get_rank() == 0 else None)
    assert os.path.exists(os.path.join(out_dir, "only_first"))          # sync=True: visible to every rank afterwards
    total = torch.tensor([float(dist.get_rank() + 1)])
    dist.all_reduce(total)
    open(os.path.join(out_dir, f"rank{dist.get_rank()}"), "w").write(str(total.item()))


def test_only_on_rank_and_all_reduce_over_two_spawned_ranks(tmp_path):
    spawn_parallel_fn(_rank_files, world_size=2, backend="gloo", master_addr="127.0.0.1", master_port="29661",
                      out_dir=str(tmp_path))
    assert (tmp_path / "only_first").read_text() == "0"
    assert (tmp_path / "rank0").read_text() == (tmp_path / "rank1").read_text() == "3.0"


def test_only_on_rank_without_a_process_group_runs_on_the_single_rank():
    calls = []

    @only_on_rank(0)
    def f(x):
        calls.append(x)
        return x * 2

    @only_on_rank(1)
    def g():
        calls.append("never")

    assert f(21) == 42 and g() is None and calls == [21]


def test_accumulation_groups_run_across_the_epoch_boundary(tmp_path):
    """Five micro-batches per epoch with two per optimizer step: the fifth of the first epoch is
    grouped with the first of the second (the micro-step counter is global), five steps in total."""
    steps = []

    class Count:
        def on_optimizer_step(self, ctx):
            steps.append((ctx.epoch, ctx.iteration))

    Trainer(_config(tmp_path, dataset=RandomTokens(n=20), n_epoch=2, grad_accum_steps=2), callbacks=[Count()]).train()
    assert steps == [(0, 2), (0, 4), (1, 6), (1, 8), (1, 10)]
    from khaosz_b200.serialization import Checkpoint

    opt = Checkpoint.load(str(tmp_path / "ck" / "epoch_1_iter_10")).extra["optimizer"]
    assert {int(st["step"]) for st in opt["state"].values()} == {5}
