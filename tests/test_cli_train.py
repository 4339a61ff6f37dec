"""End to end through the training CLI on CPU: tensor-parallel run over 2 gloo ranks writes a
checkpoint with the reference's full (unsharded) parameter names, which the dense model loads."""
import json
import os

import pytest

import torch

from khaosz_b200 import AutoRegressiveLM, AutoRegressiveLMConfig
from khaosz_b200.cli import train as train_cli
from khaosz_b200.data.storage import save_bin
from khaosz_b200.serialization import Checkpoint


def _setup(tmp_path):
    params, data = tmp_path / "params", tmp_path / "data"
    params.mkdir()
    cfg = AutoRegressiveLMConfig(vocab_size=256, dim=64, n_layers=2, norm_eps=1e-5, dim_ffn=128, tie_weight=False,
                                 max_len=32, rope_theta=1e4, n_heads=4, n_kv_heads=2)
    (params / "config.json").write_text(json.dumps(cfg.to_dict()))
    g = torch.Generator().manual_seed(0)
    save_bin(str(data / "shard_0000"), {"sequence": [torch.randint(0, 256, (32 * 40 + 1,), generator=g, dtype=torch.int32)]})
    return cfg, params, data


def _run(tmp_path, mode, nprocs, port):
    cfg, params, data = _setup(tmp_path)
    ckpt = tmp_path / f"ckpt_{mode}"
    args = train_cli.parse_args([
        "--train_type", "seq", "--data_root_path", str(data), "--param_path", str(params), "--ckpt_dir", str(ckpt),
        "--batch_per_device", "2", "--grad_accum_steps", "2", "--window_size", "32", "--num_workers", "0",
        "--no_pin_memory", "--nprocs", str(nprocs), "--parallel_mode", mode, "--backend", "gloo", "--device_type", "cpu",
        "--master_addr", "127.0.0.1", "--master_port", str(port), "--ckpt_interval", "1000000"])
    train_cli.train(args)
    dirs = sorted(d for d in os.listdir(ckpt) if d.startswith("epoch_"))
    assert dirs, "no checkpoint written"
    rows = [json.loads(line) for f in sorted(os.listdir(ckpt / "logs")) for line in open(ckpt / "logs" / f)]
    assert rows and {"loss", "lr", "tokens_per_s", "step_ms"} <= set(rows[-1])   # the metric log sits beside the checkpoints
    loaded = Checkpoint.load(str(ckpt / dirs[-1]))
    model = AutoRegressiveLM(cfg)
    model.load_state_dict(loaded.state_dict)      # full names and shapes
    assert all(torch.isfinite(v.float()).all() for v in loaded.state_dict.values())
    return loaded


def test_cli_trains_tensor_parallel_on_two_cpu_ranks(tmp_path):
    ck = _run(tmp_path, "tp", 2, 29651)
    assert ck.state_dict["layers.0.attention.q_proj.weight"].shape == (64, 64)
    assert ck.state_dict["layers.1.mlp.down.weight"].shape == (64, 128)


def test_cli_trains_fully_sharded_on_two_cpu_ranks(tmp_path):
    ck = _run(tmp_path, "fsdp_full", 2, 29653)
    assert ck.state_dict["layers.0.attention.k_proj.weight"].shape == (32, 64)


def test_cli_trains_block_sharded_on_two_cpu_ranks(tmp_path):
    ck = _run(tmp_path, "fsdp_block", 2, 29656)
    assert ck.state_dict["layers.0.attention.k_proj.weight"].shape == (32, 64)


def test_cli_trains_single_process(tmp_path):
    ck = _run(tmp_path, "none", 1, 29654)
    assert "lm_head.weight" in ck.state_dict


def test_checkpoint_of_a_tensor_parallel_run_resumes_in_a_single_process(tmp_path):
    """Weights and optimizer state written by a 2-rank tensor-parallel run load into a dense run."""
    _run(tmp_path, "tp", 2, 29655)
    first = tmp_path / "ckpt_tp"
    ckpt_dir = first / sorted(d for d in os.listdir(first) if d.startswith("epoch_"))[-1]
    assert (ckpt_dir / "optimizer.pt").exists()
    state = torch.load(ckpt_dir / "optimizer.pt", weights_only=False)
    assert state["state"][1]["exp_avg"].shape == (64, 64)       # layers.0.attention.q_proj: full shape
    out = tmp_path / "ckpt_resumed"
    args = train_cli.parse_args([
        "--train_type", "seq", "--data_root_path", str(tmp_path / "data"), "--param_path", str(ckpt_dir),
        "--ckpt_dir", str(out), "--batch_per_device", "2", "--grad_accum_steps", "2", "--window_size", "32",
        "--num_workers", "0", "--no_pin_memory", "--nprocs", "1", "--parallel_mode", "none", "--backend", "gloo",
        "--device_type", "cpu", "--master_addr", "127.0.0.1", "--master_port", "29656", "--ckpt_interval", "1000000"])
    train_cli.train(args)
    assert os.listdir(out)


@pytest.mark.parametrize("accum,optimizer", [(1, "adamw"), (2, "adamw"), (1, "muon")])
def test_cli_auto_resume_continues_from_the_newest_checkpoint(accum, optimizer, tmp_path):
    """A run that dies and is restarted with --auto_resume ends with exactly the weights of the uninterrupted run."""
    import shutil

    cfg, params, data = _setup(tmp_path)
    ckpt = tmp_path / "ckpt"
    base = ["--train_type", "seq", "--data_root_path", str(data), "--param_path", str(params), "--ckpt_dir", str(ckpt),
            "--batch_per_device", "2", "--window_size", "32", "--num_workers", "0", "--no_pin_memory", "--nprocs", "1",
            "--parallel_mode", "none", "--device_type", "cpu", "--ckpt_interval", "6", "--log_interval", "1",
            "--grad_accum_steps", str(accum), "--warmup_ratio", "0.2", "--optimizer", optimizer]
    torch.manual_seed(0)
    AutoRegressiveLM(cfg).to(torch.bfloat16).save_pretrained(str(params))     # both runs start from these weights
    assert train_cli.find_latest_checkpoint(str(ckpt)) is None
    train_cli.train(train_cli.parse_args(base + ["--auto_resume"]))        # nothing to resume: starts from --param_path
    names = sorted(d for d in os.listdir(ckpt) if d.startswith("epoch_"))
    assert names == ["epoch_0_iter_12", "epoch_0_iter_18", "epoch_0_iter_20", "epoch_0_iter_6"]
    assert train_cli.find_latest_checkpoint(str(ckpt))[0].endswith("epoch_0_iter_20")
    whole = Checkpoint.load(str(ckpt / "epoch_0_iter_20"))
    # the job "died" after iteration 6; one later checkpoint was cut off while being written
    for gone in ("epoch_0_iter_12", "epoch_0_iter_20"):
        shutil.rmtree(ckpt / gone)
    os.remove(ckpt / "epoch_0_iter_18" / "model.safetensors")
    shutil.rmtree(ckpt / "logs")
    path, meta = train_cli.find_latest_checkpoint(str(ckpt))
    # the checkpoint of iteration 6 precedes that iteration's optimizer step
    assert path.endswith("epoch_0_iter_6") and meta["iteration"] == 6 and meta["completed_iteration"] == 6 - accum
    train_cli.train(train_cli.parse_args(base + ["--auto_resume"]))
    final = Checkpoint.load(str(ckpt / "epoch_0_iter_20"))
    assert final.iteration == 20
    rows = [json.loads(line) for f in sorted(os.listdir(ckpt / "logs")) for line in open(ckpt / "logs" / f)]
    assert min(r["iter"] for r in rows) == 6 - accum + 1 and max(r["iter"] for r in rows) == 20
    for k, v in whole.state_dict.items():
        assert torch.equal(final.state_dict[k], v), k
    if optimizer == "adamw":
        opt = torch.load(ckpt / "epoch_0_iter_20" / "optimizer.pt", weights_only=False)
        assert {int(st["step"]) for st in opt["state"].values()} == {20 // accum}


def test_cli_auto_resume_twice_inside_the_second_epoch(tmp_path):
    """The iteration counter runs across epochs and across restarts: a run killed twice inside epoch 1
    picks the newest checkpoint each time (not an older one of the same epoch), continues at the right
    batch of the epoch, and ends with exactly the weights of the uninterrupted two-epoch run."""
    import shutil

    cfg, params, data = _setup(tmp_path)
    ckpt = tmp_path / "ckpt"
    base = ["--train_type", "seq", "--data_root_path", str(data), "--param_path", str(params), "--ckpt_dir", str(ckpt),
            "--batch_per_device", "2", "--window_size", "32", "--num_workers", "0", "--no_pin_memory", "--nprocs", "1",
            "--parallel_mode", "none", "--device_type", "cpu", "--ckpt_interval", "6", "--log_interval", "1",
            "--grad_accum_steps", "2", "--warmup_ratio", "0.2", "--n_epoch", "2", "--auto_resume"]
    torch.manual_seed(0)
    AutoRegressiveLM(cfg).to(torch.bfloat16).save_pretrained(str(params))
    train_cli.train(train_cli.parse_args(base))
    names = sorted((d for d in os.listdir(ckpt) if d.startswith("epoch_")), key=lambda d: int(d.rsplit("_", 1)[1]))
    assert names == ["epoch_0_iter_6", "epoch_0_iter_12", "epoch_0_iter_18", "epoch_1_iter_24", "epoch_1_iter_30",
                     "epoch_1_iter_36", "epoch_1_iter_40"]
    whole = Checkpoint.load(str(ckpt / "epoch_1_iter_40"))

    def kill_after(last_kept):
        for d in os.listdir(ckpt):
            if d.startswith("epoch_") and int(d.rsplit("_", 1)[1]) > last_kept:
                shutil.rmtree(ckpt / d)

    kill_after(24)                                   # first death: inside epoch 1, after iteration 24
    path, meta = train_cli.find_latest_checkpoint(str(ckpt))
    assert path.endswith("epoch_1_iter_24") and meta["epoch"] == 1 and meta["completed_iteration"] == 22
    train_cli.train(train_cli.parse_args(base))
    again = sorted(int(d.rsplit("_", 1)[1]) for d in os.listdir(ckpt) if d.startswith("epoch_1_"))
    assert again == [24, 28, 34, 40], again          # the resumed run keeps counting where the first one stopped
    assert Checkpoint.load(str(ckpt / "epoch_1_iter_34")).iteration == 34
    kill_after(28)                                   # second death: the newest checkpoint was written by the resumed run
    path, meta = train_cli.find_latest_checkpoint(str(ckpt))
    assert path.endswith("epoch_1_iter_28") and meta["completed_iteration"] == 26
    train_cli.train(train_cli.parse_args(base))
    final = Checkpoint.load(str(ckpt / "epoch_1_iter_40"))
    assert final.iteration == 40 and final.epoch == 1
    for k, v in whole.state_dict.items():
        assert torch.equal(final.state_dict[k], v), k
    opt = torch.load(ckpt / "epoch_1_iter_40" / "optimizer.pt", weights_only=False)
    assert {int(st["step"]) for st in opt["state"].values()} == {20}


def test_cli_lora_run_trains_adapters_only_and_saves_them(tmp_path):
    from khaosz_b200.models.components.lora import load_lora
    from khaosz_b200.serialization import load_state_dict

    cfg, params, data = _setup(tmp_path)
    torch.manual_seed(0)
    start = AutoRegressiveLM(cfg).to(torch.bfloat16)
    start.save_pretrained(str(params))
    ckpt = tmp_path / "ckpt"
    train_cli.train(train_cli.parse_args([
        "--train_type", "seq", "--data_root_path", str(data), "--param_path", str(params), "--ckpt_dir", str(ckpt),
        "--batch_per_device", "2", "--window_size", "32", "--num_workers", "0", "--no_pin_memory", "--nprocs", "1",
        "--parallel_mode", "none", "--device_type", "cpu", "--ckpt_interval", "1000", "--max_lr", "1e-2",
        "--lora_r", "4", "--lora_alpha", "8", "--lora_target_modules", "q_proj", "v_proj"]))
    adapter = ckpt / "lora_adapter"
    assert json.loads((adapter / "adapter_config.json").read_text())["r"] == 4
    weights = load_state_dict(adapter / "adapter_model.safetensors")
    assert set(k.rsplit(".", 1)[1] for k in weights) == {"lora_A", "lora_B"} and len(weights) == 2 * 2 * cfg.n_layers
    assert weights["layers.0.attention.q_proj.lora_B"].float().abs().sum() > 0        # B starts at zero: it has trained
    final = Checkpoint.load(str(ckpt / "epoch_0_iter_20")).state_dict
    base = start.state_dict()
    assert torch.equal(final["layers.0.attention.q_proj.weight"], base["layers.0.attention.q_proj.weight"])   # frozen
    assert not torch.equal(final["layers.0.attention.k_proj.weight"], base["layers.0.attention.k_proj.weight"])
    fresh = AutoRegressiveLM(cfg).to(torch.bfloat16)
    fresh.load_state_dict(base)
    assert load_lora(fresh, str(adapter)).r == 4                                      # the adapters load onto the base model
    with pytest.raises(ValueError, match="LoRA"):
        train_cli.train(train_cli.parse_args([
            "--train_type", "seq", "--data_root_path", str(data), "--param_path", str(params), "--ckpt_dir", str(ckpt),
            "--nprocs", "2", "--parallel_mode", "tp", "--lora_r", "4"]))


def _two_rank_config(tmp_path, mode):
    from conftest import RandomTokens, tiny_config
    from khaosz_b200 import TrainConfig

    cfg = tiny_config(n_heads=4, n_kv_heads=2)
    return TrainConfig(model_fn=_TinyFactory(cfg), strategy="seq", dataset=RandomTokens(n=48),
                       optimizer_fn=_adamw, scheduler_fn=_cosine, batch_per_device=4, grad_accum_steps=2,
                       ckpt_dir=str(tmp_path / "ck"), log_dir=str(tmp_path / "logs"), ckpt_interval=1000, log_interval=1,
                       device_type="cpu", backend="gloo", nprocs=2, parallel_mode=mode, master_addr="127.0.0.1",
                       master_port="29662" if mode == "ddp" else "29663", val_split=0.25, val_step=1,
                       metrics=["loss", "lr", "val_loss", "tokens_per_s"])


class _TinyFactory:
    """Picklable model factory (the trainer spawns its ranks)."""

    def __init__(self, cfg):
        self.cfg = cfg

    def __call__(self):
        torch.manual_seed(0)
        return AutoRegressiveLM(self.cfg)


def _adamw(model):
    from khaosz_b200.trainer import FusedAdamW

    return FusedAdamW(model.parameters(), lr=1e-3)


def _cosine(opt):
    from khaosz_b200.trainer import SchedulerFactory

    return SchedulerFactory.create(opt, "cosine", warmup_steps=2, lr_decay_steps=20)


@pytest.mark.parametrize("mode", ["ddp", "fsdp", "fsdp_zero1"])
def test_trainer_with_validation_on_two_ranks(tmp_path, mode):
    from khaosz_b200.trainer import Trainer

    Trainer(_two_rank_config(tmp_path, mode)).train()
    rows = [json.loads(line) for f in sorted(os.listdir(tmp_path / "logs")) for line in open(tmp_path / "logs" / f)]
    assert rows and rows[-1]["val_loss"] > 0 and rows[-1]["tokens_per_s"] > 0
    # 36 training samples over two ranks, four per micro-batch: five iterations each (the last one padded)
    final = sorted(d for d in os.listdir(tmp_path / "ck") if d.startswith("epoch_"))[-1]
    assert (tmp_path / "ck" / final / "optimizer.pt").exists()


def test_resuming_a_lora_run_keeps_the_adapters(tmp_path):
    cfg, params, data = _setup(tmp_path)
    torch.manual_seed(0)
    AutoRegressiveLM(cfg).to(torch.bfloat16).save_pretrained(str(params))
    ckpt = tmp_path / "ckpt"
    base = ["--train_type", "seq", "--data_root_path", str(data), "--param_path", str(params), "--ckpt_dir", str(ckpt),
            "--batch_per_device", "2", "--window_size", "32", "--num_workers", "0", "--no_pin_memory", "--nprocs", "1",
            "--parallel_mode", "none", "--device_type", "cpu", "--ckpt_interval", "6", "--max_lr", "1e-2",
            "--lora_r", "4", "--lora_alpha", "8", "--warmup_ratio", "0.2"]
    train_cli.train(train_cli.parse_args(base))
    whole = Checkpoint.load(str(ckpt / "epoch_0_iter_20")).state_dict
    import shutil

    for gone in ("epoch_0_iter_12", "epoch_0_iter_18", "epoch_0_iter_20", "lora_adapter"):
        shutil.rmtree(ckpt / gone)
    train_cli.train(train_cli.parse_args(base + ["--auto_resume"]))
    resumed = Checkpoint.load(str(ckpt / "epoch_0_iter_20")).state_dict
    key = "layers.0.attention.q_proj.lora_B"
    assert float(whole[key].float().abs().sum()) > 0
    for k, v in whole.items():                        # adapters included: the restart continued, it did not start them over
        assert torch.equal(resumed[k], v), k


@pytest.mark.parametrize("mode,port", [("ddp", 29692), ("fsdp", 29693), ("tp", 29694), ("fsdp_zero1", 29696)])
def test_auto_resume_is_exact_on_two_ranks(mode, port, tmp_path):
    """A killed and restarted two-rank run (data parallel, sharded optimizer, tensor parallel) ends with the
    weights of the uninterrupted one."""
    import shutil

    cfg, params, data = _setup(tmp_path)
    torch.manual_seed(0)
    AutoRegressiveLM(cfg).to(torch.bfloat16).save_pretrained(str(params))
    ckpt = tmp_path / "ckpt"
    base = ["--train_type", "seq", "--data_root_path", str(data), "--param_path", str(params), "--ckpt_dir", str(ckpt),
            "--batch_per_device", "2", "--window_size", "32", "--num_workers", "0", "--no_pin_memory", "--nprocs", "2",
            "--parallel_mode", mode, "--backend", "gloo", "--device_type", "cpu", "--master_addr", "127.0.0.1",
            "--master_port", str(port), "--ckpt_interval", "6", "--warmup_ratio", "0.2"]
    train_cli.train(train_cli.parse_args(base))
    dirs = sorted((d for d in os.listdir(ckpt) if d.startswith("epoch_")), key=lambda d: int(d.rsplit("_", 1)[1]))
    final = dirs[-1]
    whole = Checkpoint.load(str(ckpt / final)).state_dict
    for gone in dirs[1:]:
        shutil.rmtree(ckpt / gone)
    assert dirs[0] == "epoch_0_iter_6"
    train_cli.train(train_cli.parse_args(base + ["--auto_resume"]))
    resumed = Checkpoint.load(str(ckpt / final)).state_dict
    for k, v in whole.items():
        assert torch.equal(resumed[k], v), k


@pytest.mark.parametrize("mode", ["ddp", "fsdp", "fsdp_zero1", "fsdp_full", "tp"])
def test_parallel_modes_degrade_to_a_single_process(mode, tmp_path):
    ck = _run(tmp_path, mode, 1, 29695)
    assert ck.iteration == 20 and "layers.1.mlp.down.weight" in ck.state_dict
