import json
import os

import pytest
import torch
import torch.nn.functional as F

from conftest import RandomTokens, tiny_config
from khaosz_b200 import AutoRegressiveLM, TrainConfig
from khaosz_b200.models.components.block import DecoderBlock
from khaosz_b200.serialization import Checkpoint
from khaosz_b200.trainer import (CallbackFactory, FusedAdamW, GradientCheckpointingCallback, Muon, SchedulerFactory,
                                 StrategyFactory, Trainer, get_logprobs)
from khaosz_b200.trainer.metrics import grad_nan_num, grad_norm


def _config(tmp_path, dataset=None, **over):
    cfg = tiny_config()
    base = dict(model_fn=lambda: AutoRegressiveLM(cfg), strategy="seq", dataset=dataset or RandomTokens(),
                optimizer_fn=lambda m: FusedAdamW(m.parameters(), lr=1e-3),
                scheduler_fn=lambda o: SchedulerFactory.create(o, "cosine", warmup_steps=2, lr_decay_steps=20),
                batch_per_device=4, ckpt_dir=str(tmp_path / "ck"), log_dir=str(tmp_path / "logs"), ckpt_interval=1000,
                log_interval=1, device_type="cpu", n_epoch=1)
    base.update(over)
    return TrainConfig(**base)


@pytest.mark.parametrize("accum", [1, 2, 4])
def test_trainer_end_to_end(tmp_path, accum):
    Trainer(_config(tmp_path, grad_accum_steps=accum)).train()
    ck = tmp_path / "ck" / "epoch_0_iter_8"
    assert (ck / "model.safetensors").exists() and (ck / "optimizer.pt").exists() and (ck / "scheduler.pt").exists()
    rows = [json.loads(l) for l in open(tmp_path / "logs" / "epoch_0_iter_8_metric.jsonl")]
    assert len(rows) == 8 and {"timestamp", "epoch", "iter", "loss", "lr"} <= set(rows[0])
    sched = torch.load(ck / "scheduler.pt", weights_only=False)
    assert sched["last_epoch"] == 8 // accum and sched["warmup_steps"] == 2


def test_callbacks_all_fire_and_loss_drops(tmp_path):
    class Spy:
        def __init__(self):
            self.calls, self.losses = [], []

        def __getattr__(self, name):
            if name.startswith("on_"):
                def hook(ctx, name=name):
                    self.calls.append(name)
                    if name == "on_batch_end":
                        self.losses.append(ctx.loss)
                return hook
            raise AttributeError(name)

    spy = Spy()
    t = Trainer(_config(tmp_path, dataset=RandomTokens(n=64), n_epoch=3, max_grad_norm=1.0,
                        optimizer_fn=lambda m: FusedAdamW(m.parameters(), lr=5e-3)), callbacks=[spy])
    assert [type(c).__name__ for c in t.callbacks[:6]] == [
        "GradientCheckpointingCallback", "CheckpointCallback", "MetricLoggerCallback", "ProgressBarCallback",
        "GradientClippingCallback", "ValidationCallback"]
    t.train()
    for hook in ("on_train_begin", "on_train_end", "on_epoch_begin", "on_epoch_end", "on_batch_begin", "on_batch_end",
                 "on_optimizer_step"):
        assert hook in spy.calls
    assert "on_error" not in spy.calls and spy.calls.count("on_batch_end") == 48
    assert sum(spy.losses[-8:]) < sum(spy.losses[:8])


def test_fault_injection_emergency_checkpoint_and_resume(tmp_path):
    ds = RandomTokens(n=40, fail_at=11)  # third batch of 4 raises
    with pytest.raises(RuntimeError, match="injected"):
        Trainer(_config(tmp_path, dataset=ds)).train()
    ck = tmp_path / "ck" / "epoch_0_iter_2"
    assert ck.exists() and json.loads((ck / "meta.json").read_text())["iteration"] == 2
    Trainer(_config(tmp_path, dataset=RandomTokens(n=40), start_epoch=0, start_batch=2)).train(resume_dir=str(ck))
    final = tmp_path / "ck" / "epoch_0_iter_10"
    assert json.loads((final / "meta.json").read_text())["iteration"] == 10
    back = Checkpoint.load(str(final))
    assert "optimizer" in back.extra and "scheduler" in back.extra


def test_validation_split_and_metrics(tmp_path):
    cfg = _config(tmp_path, dataset=RandomTokens(n=40), val_split=0.2, val_step=1, metrics=["loss", "lr", "val_loss", "grad_norm"])
    Trainer(cfg).train()
    files = os.listdir(tmp_path / "logs")
    rows = [json.loads(l) for l in open(tmp_path / "logs" / files[0])]
    assert rows[-1]["val_loss"] > 0 and isinstance(rows[-1]["grad_norm"], dict)


def test_gradient_checkpointing_callback():
    model = AutoRegressiveLM(tiny_config()).eval()
    ids = torch.randint(0, 300, (2, 8))
    with torch.no_grad():
        ref = model(ids)["logits"]
    cb = GradientCheckpointingCallback([DecoderBlock])
    model.apply(cb._enable)
    assert all(hasattr(l, "_original_forward") for l in model.layers)
    with torch.no_grad():
        assert torch.equal(model(ids)["logits"], ref)
    model.train()
    model(ids)["logits"].sum().backward()
    assert all(p.grad is not None for p in model.parameters())
    model.apply(cb._disable)
    assert not any(hasattr(l, "_original_forward") for l in model.layers)


# ---- schedulers ----
def test_cosine_scheduler_curve_and_state():
    opt = torch.optim.SGD([torch.nn.Parameter(torch.zeros(1))], lr=1.0)
    s = SchedulerFactory.create(opt, "cosine", warmup_steps=4, lr_decay_steps=10, min_rate=0.1)
    lrs = [opt.param_groups[0]["lr"]]
    for _ in range(16):
        opt.step()
        s.step()
        lrs.append(opt.param_groups[0]["lr"])
    assert lrs[0] == pytest.approx(0.1) and lrs[2] == pytest.approx(0.5) and lrs[4] == pytest.approx(1.0)
    assert lrs[9] == pytest.approx(0.5) and lrs[14] == pytest.approx(0.1) and lrs[16] == pytest.approx(0.1)
    state = s.state_dict()
    assert state["warmup_steps"] == 4 and state["min_rate"] == 0.1
    opt2 = torch.optim.SGD([torch.nn.Parameter(torch.zeros(1))], lr=1.0)
    s2 = SchedulerFactory.create(opt2, "cosine", warmup_steps=1, lr_decay_steps=1)
    s2.load_state_dict(state)
    assert s2.last_epoch == 16 and s2.warmup_steps == 4 and s2.get_last_lr() == s.get_last_lr()


def test_sgdr_scheduler_restarts():
    opt = torch.optim.SGD([torch.nn.Parameter(torch.zeros(1))], lr=1.0)
    s = SchedulerFactory.create(opt, "sgdr", warmup_steps=2, cycle_length=4, min_rate=0.0, t_mult=2)
    lrs = []
    for _ in range(15):
        opt.step()
        s.step()
        lrs.append(opt.param_groups[0]["lr"])
    assert lrs[1] == pytest.approx(1.0) and lrs[5] == pytest.approx(1.0) and lrs[13] == pytest.approx(1.0)  # restarts
    assert lrs[3] == pytest.approx(0.5)
    assert set(SchedulerFactory.available_types()) >= {"cosine", "sgdr"}
    with pytest.raises(ValueError):
        SchedulerFactory.create(opt, "linear")


# ---- strategies: loss values against plain PyTorch ----
def test_seq_and_sft_loss_values(tiny_model):
    ids = torch.randint(0, 300, (2, 9))
    batch = {"input_ids": ids[:, :-1], "target_ids": ids[:, 1:]}
    logits = tiny_model(batch["input_ids"])["logits"]
    want = F.cross_entropy(logits.flatten(0, 1), batch["target_ids"].flatten(), label_smoothing=0.1)
    got = StrategyFactory.create("seq", tiny_model, "cpu", label_smoothing=0.1)(batch)
    assert got.item() == pytest.approx(want.item(), rel=1e-5)
    mask = torch.zeros(2, 8, dtype=torch.bool)
    mask[:, 4:] = True
    want = F.cross_entropy(logits[:, 4:].flatten(0, 1), batch["target_ids"][:, 4:].flatten())
    got = StrategyFactory.create("sft", tiny_model, "cpu")({**batch, "loss_mask": mask})
    assert got.item() == pytest.approx(want.item(), rel=1e-5)


class _NoneExec:
    def unwrap_model(self, m):
        return m.state_dict()


def test_dpo_loss_value(tiny_model):
    cfg = tiny_config()
    strat = StrategyFactory.create("dpo", tiny_model, "cpu", executor=_NoneExec(), model_fn=lambda: AutoRegressiveLM(cfg),
                                   beta=0.1, reduction="sum")
    g = torch.Generator().manual_seed(0)
    batch = {"chosen": torch.randint(0, 300, (2, 10), generator=g), "rejected": torch.randint(0, 300, (2, 10), generator=g),
             "chosen_mask": torch.ones(2, 10, dtype=torch.bool), "rejected_mask": torch.ones(2, 10, dtype=torch.bool)}
    loss0 = strat(batch)
    assert loss0.item() == pytest.approx(0.6931, abs=1e-3)  # policy == reference -> log 2
    with torch.no_grad():
        for p in tiny_model.parameters():
            p.add_(0.01 * torch.randn_like(p))

    def lp(model, ids):
        out = torch.log_softmax(model(ids[:, :-1])["logits"].float(), -1)
        return out.gather(-1, ids[:, 1:, None]).squeeze(-1).sum(-1)

    margin = (lp(tiny_model, batch["chosen"]) - lp(tiny_model, batch["rejected"])) - (
        lp(strat.ref_model, batch["chosen"]) - lp(strat.ref_model, batch["rejected"]))
    want = -F.logsigmoid(0.1 * margin).mean()
    got = strat(batch)
    assert got.item() == pytest.approx(want.item(), rel=1e-4)
    got.backward()
    assert not any(p.requires_grad for p in strat.ref_model.parameters())


def test_grpo_loss_and_ref_sync(tiny_model):
    cfg = tiny_config()
    strat = StrategyFactory.create("grpo", tiny_model, "cpu", executor=_NoneExec(),
                                   model_fn=lambda: AutoRegressiveLM(cfg), group_size=4, sync_interval=2, kl_coef=0.0)
    g = torch.Generator().manual_seed(0)
    batch = {"prompts": torch.randint(0, 300, (2, 5), generator=g), "responses": torch.randint(0, 300, (2, 4, 6), generator=g),
             "masks": torch.ones(2, 4, 6, dtype=torch.bool), "rewards": torch.rand(2, 4, generator=g)}
    loss = strat(batch)
    assert loss.item() == pytest.approx(0.0, abs=1e-5)  # ratio == 1, advantages sum to zero per group
    loss.backward()
    with torch.no_grad():
        tiny_model.norm.weight.add_(1.0)
    strat(batch)  # second call: sync_interval hit -> reference refreshed
    assert torch.equal(strat.ref_model.norm.weight, tiny_model.norm.weight)
    flat = {"prompts": batch["prompts"], "responses": batch["responses"].reshape(2, 24),
            "masks": batch["masks"].reshape(2, 24), "rewards": torch.rand(2, 24, generator=g)}
    assert torch.isfinite(strat(flat))


def test_get_logprobs_reductions(tiny_model):
    ids = torch.randint(0, 300, (2, 7))
    mask = torch.ones(2, 7, dtype=torch.bool)
    mask[1, 4:] = False
    none = get_logprobs(tiny_model, ids, mask, "none")
    assert none.shape == (2, 6) and (none[1, 3:] == 0).all()
    assert torch.allclose(get_logprobs(tiny_model, ids, mask, "sum"), none.sum(-1))
    assert torch.allclose(get_logprobs(tiny_model, ids, mask, "mean")[1], none[1].sum() / 3)
    with pytest.raises(ValueError):
        get_logprobs(tiny_model, ids, mask, "max")


def test_muon_and_metrics(tiny_model):
    opt = Muon(tiny_model.parameters(), lr=1e-2)
    ids = torch.randint(0, 300, (2, 9))
    losses = []
    for _ in range(5):
        loss = F.cross_entropy(tiny_model(ids[:, :-1])["logits"].flatten(0, 1), ids[:, 1:].flatten())
        loss.backward()
        norms = grad_norm(tiny_model)
        opt.step()
        opt.zero_grad()
        losses.append(loss.item())
    assert losses[-1] < losses[0] and all(v >= 0 for v in norms.values())
    assert set(grad_nan_num(tiny_model).values()) == {0}
    assert set(CallbackFactory.list_registered()) >= {"gradient_clipping", "gradient_checkpointing", "checkpoint",
                                                      "progress_bar", "metric_logger", "validation"}


def test_device_health_callback_raises_into_the_error_path():
    """A device-side error code surfaces at the optimizer step as an exception (fake error word)."""
    from khaosz_b200.trainer.callbacks import CallbackFactory

    calls = []

    def check():
        calls.append(1)
        if len(calls) == 2:
            raise RuntimeError("device-side kernel error: timeout waiting for a peer flag")

    cb = CallbackFactory.create("device_health", check=check)
    cb.on_optimizer_step(None)
    with pytest.raises(RuntimeError, match="peer flag"):
        cb.on_optimizer_step(None)


def test_device_health_probes_after_the_step_and_at_the_end():
    """After an optimizer step the error word is probed without blocking and polled on the following
    batches; the end of training checks once more, so a failure in the last step is not lost."""
    from types import SimpleNamespace

    from khaosz_b200.trainer.callbacks import CallbackFactory

    log_ = []

    class FakeProbe:
        def post(self):
            log_.append("post")

        def poll(self):
            log_.append("poll")
            if log_.count("poll") == 3:
                raise RuntimeError("device-side kernel error: timeout waiting for a peer flag")

    cb = CallbackFactory.create("device_health", check=lambda: log_.append("check"), probe=FakeProbe())
    ctx = SimpleNamespace(kwargs={})
    cb.on_batch_begin(ctx)                       # nothing stepped yet: poll only
    cb.on_optimizer_step(ctx)                    # synchronous check before the update
    cb.on_batch_begin(ctx)                       # the step is enqueued: probe behind it, then poll
    assert log_ == ["poll", "check", "post", "poll"]
    with pytest.raises(RuntimeError, match="peer flag"):
        cb.on_batch_begin(ctx)
    cb.on_train_end(ctx)
    assert log_[-1] == "check"
    ctx.kwargs["error"] = RuntimeError("x")      # already failing: the end-of-training check stays quiet
    n = len(log_)
    cb.on_train_end(ctx)
    assert len(log_) == n


def test_no_emergency_checkpoint_after_a_device_side_failure(tmp_path):
    """A KernelError (a collective that gave up) must not leave a checkpoint that --auto_resume would pick."""
    from types import SimpleNamespace

    from khaosz_b200.ops._lib import KernelError
    from khaosz_b200.serialization import find_latest_checkpoint
    from khaosz_b200.trainer.callbacks import CallbackFactory

    model = torch.nn.Linear(4, 4)
    ex = SimpleNamespace(unwrap_model=lambda m: m.state_dict(), grad_accum_steps=1)
    cb = CallbackFactory.create("checkpoint", str(tmp_path), 100, weight_only=True)
    ctx = SimpleNamespace(kwargs={"error": KernelError("device-side kernel error: timeout waiting for a peer flag")},
                          executor=ex, model=model, iteration=7, epoch=0, model_config={}, checkpoint=None)
    cb.on_error(ctx)
    assert find_latest_checkpoint(str(tmp_path)) is None
    ctx.kwargs["error"] = ValueError("host-side failure")       # any other failure still writes the emergency checkpoint
    cb.on_error(ctx)
    assert find_latest_checkpoint(str(tmp_path))[0].endswith("epoch_0_iter_7")


def test_trace_ranges_are_noops_without_cuda():
    from khaosz_b200.utils import enable_tracing, trace_range

    enable_tracing(True)
    try:
        with trace_range("x"):
            pass
    finally:
        enable_tracing(False)
    with trace_range("y"):
        pass


def test_throughput_callback_reports_step_time_and_tokens_per_second(tmp_path):
    from types import SimpleNamespace

    from khaosz_b200.trainer.callbacks import batch_tokens

    assert batch_tokens({"input_ids": torch.zeros(4, 16), "target_ids": torch.zeros(4, 16)}) == 64
    assert batch_tokens({"chosen": torch.zeros(2, 8), "rejected": torch.zeros(2, 8), "chosen_mask": torch.zeros(2, 8)}) == 32
    ticks = iter([10.0, 10.5, 11.5])
    cb = CallbackFactory.create("throughput", clock=lambda: next(ticks), use_cuda=False)
    ctx = SimpleNamespace(kwargs={"batch_tokens": 100}, world_size=2,
                          dataloader=SimpleNamespace(sampler=SimpleNamespace(num_replicas=2)))
    for _ in range(3):          # three optimizer steps of two micro-batches each
        cb.on_batch_end(ctx)
        cb.on_batch_end(ctx)
        cb.on_optimizer_step(ctx)
    assert ctx.kwargs["step_ms"] == pytest.approx(1000.0)
    assert ctx.kwargs["tokens_per_s"] == pytest.approx(200 * 2 / 1.0)

    # through the trainer: the metric log carries both figures
    Trainer(_config(tmp_path, metrics=["loss", "tokens_per_s", "step_ms"])).train()
    files = os.listdir(tmp_path / "logs")
    rows = [json.loads(l) for l in open(tmp_path / "logs" / files[0])]
    assert rows[-1]["tokens_per_s"] > 0 and rows[-1]["step_ms"] > 0


def test_throughput_callback_device_detection(monkeypatch):
    from types import SimpleNamespace

    monkeypatch.setattr(torch.cuda, "is_available", lambda: True)
    monkeypatch.setenv("LOCAL_DEVICE", "cpu")       # a CPU rank on a box that has GPUs
    cb = CallbackFactory.create("throughput")
    ctx = SimpleNamespace(kwargs={"batch_tokens": 8}, world_size=1, dataloader=None)
    cb.on_batch_end(ctx)
    cb.on_optimizer_step(ctx)
    cb.on_batch_end(ctx)
    cb.on_optimizer_step(ctx)
    assert cb._use_cuda is False and ctx.kwargs["tokens_per_s"] > 0


def test_iteration_counter_runs_across_epochs(tmp_path):
    """Two epochs of five micro-batches: the final checkpoint is ``epoch_1_iter_10`` (the counter is
    global, not per epoch; pinned by the reference's tests/trainer/test_early_stopping.py:46-57)."""
    Trainer(_config(tmp_path, dataset=RandomTokens(n=20), n_epoch=2, grad_accum_steps=2)).train()
    final = tmp_path / "ck" / "epoch_1_iter_10"
    assert json.loads((final / "meta.json").read_text())["iteration"] == 10


def test_fully_masked_batches_give_zero_loss_and_zero_gradients(tiny_model):
    ids = torch.randint(0, 300, (2, 9))
    strat = StrategyFactory.create("sft", tiny_model, "cpu")
    loss = strat({"input_ids": ids[:, :-1], "target_ids": ids[:, 1:], "loss_mask": torch.zeros(2, 8, dtype=torch.bool)})
    assert loss.item() == 0.0
    loss.backward()
    assert all(p.grad is None or float(p.grad.abs().sum()) == 0.0 for p in tiny_model.parameters())
    partly = torch.zeros(2, 8, dtype=torch.bool)
    partly[0, 3:] = True
    loss = strat({"input_ids": ids[:, :-1], "target_ids": ids[:, 1:], "loss_mask": partly})
    logits = tiny_model(ids[:, :-1])["logits"]
    want = F.cross_entropy(logits[0, 3:].float(), ids[0, 4:])
    assert loss.item() == pytest.approx(want.item(), rel=1e-5)
