import json
import os

import pytest
import torch

from khaosz_b200.data import (DatasetFactory, MmapStore, ResumableDistributedSampler, StoreFactory, detect_format,
                              load_bin, save_bin)
from khaosz_b200.parallel import spawn_parallel_fn
from khaosz_b200.serialization import Checkpoint


def _make_bin(path, n=100, keys=("sequence",), dtype=torch.int32):
    save_bin(str(path), {k: [torch.arange(n, dtype=dtype)] for k in keys})


def test_bin_roundtrip_and_multi_segment(tmp_path):
    save_bin(str(tmp_path / "s0"), {"sequence": [torch.arange(10, dtype=torch.int32), torch.arange(10, 30, dtype=torch.int32)]})
    meta = json.loads((tmp_path / "s0" / "meta.json").read_text())
    assert meta["sequence"] == {"shape": [30], "dtype": "int32"}
    assert torch.equal(load_bin(str(tmp_path / "s0"))["sequence"][0], torch.arange(30, dtype=torch.int32))
    save_bin(str(tmp_path / "s1"), {"sequence": [torch.arange(30, 50, dtype=torch.int32)]})
    store = MmapStore()
    store.load(str(tmp_path))
    assert len(store) == 50 and store.keys == ["sequence"]
    assert store.fetch(25, 35, "sequence").tolist() == list(range(25, 35))  # crosses the shard boundary
    assert store.fetch(10, 10, "sequence").numel() == 0
    assert set(store.fetch(0, 3, ["sequence"]).keys()) == {"sequence"}


def test_store_errors(tmp_path):
    store = MmapStore()
    with pytest.raises(RuntimeError, match="not loaded"):
        store.fetch(0, 1, "sequence")
    _make_bin(tmp_path / "d", 50)
    store.load(str(tmp_path / "d"))
    for bad in ((50, 50), (-1, 3), (0, 51)):
        with pytest.raises(ValueError, match="out of bounds"):
            store.fetch(*bad, "sequence")
    with pytest.raises(ValueError, match="Unknown component"):
        StoreFactory.create("parquet")


def test_detect_format(tmp_path):
    empty = tmp_path / "empty"
    empty.mkdir()
    with pytest.raises(FileNotFoundError, match="No supported"):
        detect_format(str(empty))
    f = tmp_path / "x.txt"
    f.write_text("hi")
    with pytest.raises(ValueError, match="Unsupported"):
        detect_format(str(f))
    _make_bin(tmp_path / "b")
    assert detect_format(str(tmp_path / "b")) == "bin"
    (tmp_path / "b" / "z.h5").write_bytes(b"")
    assert detect_format(str(tmp_path / "b")) == "h5"  # h5 wins


@pytest.mark.parametrize("n,window,stride", [(100, 10, 10), (100, 16, 4), (57, 8, 8), (11, 10, 1)])
def test_dataset_windows(tmp_path, n, window, stride):
    _make_bin(tmp_path / "d", n)
    ds = DatasetFactory.load("seq", str(tmp_path / "d"), window, stride)
    assert ds.count == n and len(ds) == (n - 1 - window) // stride + 1
    item = ds[0]
    assert item["input_ids"].dtype == torch.long and item["input_ids"].shape == (window,)
    assert torch.equal(item["target_ids"], item["input_ids"] + 1)
    last = ds[len(ds) - 1]
    assert last["target_ids"][-1].item() <= n - 1


def test_dataset_short_and_unloaded(tmp_path):
    _make_bin(tmp_path / "d", 5)
    ds = DatasetFactory.load("seq", str(tmp_path / "d"), 10)
    assert len(ds) == 0 and ds.count == 5
    fresh = DatasetFactory.create("seq", 4, 4)
    with pytest.raises(RuntimeError, match="not loaded"):
        fresh.get_index(0)
    assert len(fresh) == 0 and fresh.keys == []
    assert set(DatasetFactory.available_types()) >= {"seq", "sft", "dpo", "grpo"}


def test_sft_dpo_grpo_dtypes_and_missing_keys(tmp_path):
    save_bin(str(tmp_path / "sft"), {"sequence": [torch.arange(40, dtype=torch.int32)],
                                     "loss_mask": [torch.ones(40, dtype=torch.int32)]})
    item = DatasetFactory.load("sft", str(tmp_path / "sft"), 8)[1]
    assert item["loss_mask"].dtype == torch.bool and item["loss_mask"].shape == (8,)
    keys = ["chosen", "rejected", "chosen_mask", "rejected_mask"]
    save_bin(str(tmp_path / "dpo"), {k: [torch.arange(40, dtype=torch.int32)] for k in keys})
    item = DatasetFactory.load("dpo", str(tmp_path / "dpo"), 8)[0]
    assert item["chosen"].dtype == torch.long and item["rejected_mask"].dtype == torch.bool
    save_bin(str(tmp_path / "grpo"), {"prompts": [torch.arange(40, dtype=torch.int32)],
                                      "responses": [torch.arange(40, dtype=torch.int32)],
                                      "masks": [torch.ones(40, dtype=torch.int32)],
                                      "rewards": [torch.rand(40)]})
    item = DatasetFactory.load("grpo", str(tmp_path / "grpo"), 8)[0]
    assert (item["prompts"].dtype, item["masks"].dtype, item["rewards"].dtype) == (torch.long, torch.bool, torch.float32)
    _make_bin(tmp_path / "seqonly", 40)
    with pytest.raises(KeyError):
        DatasetFactory.load("sft", str(tmp_path / "seqonly"), 8)


def test_sampler_determinism_epochs_and_resume():
    data = list(range(20))
    a = list(ResumableDistributedSampler(data, seed=1, num_replicas=1, rank=0))
    b = list(ResumableDistributedSampler(data, seed=1, num_replicas=1, rank=0))
    assert a == b and sorted(a) == data
    s = ResumableDistributedSampler(data, seed=1, num_replicas=1, rank=0)
    e0, e1 = list(s), list(s)
    assert e0 != e1 and sorted(e1) == data  # epoch advanced automatically
    resumed = ResumableDistributedSampler(data, seed=1, start_iter=5, num_replicas=1, rank=0)
    assert len(resumed) == 15 and list(resumed) == a[5:]
    r0 = list(ResumableDistributedSampler(data, seed=3, num_replicas=2, rank=0))
    r1 = list(ResumableDistributedSampler(data, seed=3, num_replicas=2, rank=1))
    assert sorted(r0 + r1) == data


def test_checkpoint_roundtrip(tmp_path):
    sd = {"w": torch.randn(3, 4), "b": torch.zeros(2)}
    ck = Checkpoint(state_dict=sd, epoch=2, iteration=7, extra={"optimizer": {"lr": 0.1}, "scheduler": {"last_epoch": 3}},
                    config={"dim": 4})
    ck.save(str(tmp_path / "ck"))
    for name in ("meta.json", "config.json", "model.safetensors", "optimizer.pt", "scheduler.pt"):
        assert (tmp_path / "ck" / name).exists()
    back = Checkpoint.load(str(tmp_path / "ck"))
    assert back.epoch == 2 and back.iteration == 7 and back.config == {"dim": 4}
    assert torch.equal(back.state_dict["w"], sd["w"]) and back.extra["optimizer"] == {"lr": 0.1}
    assert json.loads((tmp_path / "ck" / "meta.json").read_text())["iteration"] == 7


def _two_rank_ckpt(path):
    import torch.distributed as dist

    rank = dist.get_rank()
    Checkpoint(state_dict={"w": torch.full((2,), float(rank))}, iteration=3).save(path)
    dist.barrier()
    got = Checkpoint.load(path, broadcast=True)
    assert got.iteration == 3 and torch.equal(got.state_dict["w"], torch.zeros(2))  # rank 0 wrote it


def test_checkpoint_two_ranks(tmp_path):
    spawn_parallel_fn(_two_rank_ckpt, world_size=2, backend="gloo", master_addr="127.0.0.1", master_port="29611",
                      path=str(tmp_path / "ck2"))


def test_checkpoint_files_are_written_atomically_and_meta_comes_last(tmp_path, monkeypatch):
    import khaosz_b200.serialization as ser

    order = []
    real_replace = os.replace

    def spy(src, dst):
        order.append(os.path.basename(str(dst)))
        assert str(src).endswith(".tmp") and os.path.exists(src)
        real_replace(src, dst)

    monkeypatch.setattr(ser.os, "replace", spy)
    ck = Checkpoint(state_dict={"w": torch.ones(3)}, epoch=1, iteration=7, extra={"optimizer": {"lr": 0.1}},
                    config={"dim": 8}, meta={"completed_iteration": 6})
    ck.save(str(tmp_path / "ck"))
    assert order[-1] == "meta.json" and set(order) == {"config.json", "model.safetensors", "optimizer.pt", "meta.json"}
    assert not [p for p in os.listdir(tmp_path / "ck") if p.endswith(".tmp")]
    meta = json.loads((tmp_path / "ck" / "meta.json").read_text())
    assert meta["epoch"] == 1 and meta["iteration"] == 7 and meta["completed_iteration"] == 6 and "timestamp" in meta

    # a write that dies half-way leaves the previous file intact and no debris
    def boom(tmp):
        tmp.write_text("partial")
        raise OSError("disk full")

    with pytest.raises(OSError):
        ser._atomically(tmp_path / "ck" / "meta.json", boom)
    assert json.loads((tmp_path / "ck" / "meta.json").read_text())["iteration"] == 7
    assert not [p for p in os.listdir(tmp_path / "ck") if p.endswith(".tmp")]
