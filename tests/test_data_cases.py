"""Case-by-case behaviour of the storage layer, the windowed datasets and the resumable sampler
(the behaviours the reference pins in ``tests/data/test_dataset.py`` and ``tests/data/test_sampler.py``)."""
import json

import pytest
import torch
from torch.utils.data import DataLoader

from khaosz_b200.data import (DatasetFactory, H5Store, MmapStore, ResumableDistributedSampler, StoreFactory,
                              detect_format, load_bin, save_bin)


def _ramp(path, n, keys=("sequence",), dtype=torch.int32, start=0):
    save_bin(str(path), {k: [torch.arange(start, start + n, dtype=dtype)] for k in keys})


# ---- bin files --------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.int16, torch.int32, torch.int64, torch.float32, torch.uint8])
def test_bin_round_trip_keeps_dtype_and_values(tmp_path, dtype):
    data = (torch.arange(40) % 100).to(dtype)
    save_bin(str(tmp_path / "s"), {"sequence": [data[:15], data[15:]]})
    back = load_bin(str(tmp_path / "s"))["sequence"]
    assert len(back) == 1 and back[0].dtype == dtype and torch.equal(back[0], data)   # segments are concatenated on disk
    meta = json.loads((tmp_path / "s" / "meta.json").read_text())
    assert meta["sequence"]["shape"] == [40]


def test_bin_keeps_several_keys_apart(tmp_path):
    save_bin(str(tmp_path / "s"), {"sequence": [torch.arange(10, dtype=torch.int32)],
                                   "loss_mask": [torch.ones(10, dtype=torch.int32)]})
    assert sorted(p.name for p in (tmp_path / "s").iterdir()) == ["loss_mask.bin", "meta.json", "sequence.bin"]
    back = load_bin(str(tmp_path / "s"))
    assert back["loss_mask"][0].sum() == 10 and back["sequence"][0][-1] == 9


def test_detect_format_on_files_and_trees(tmp_path):
    _ramp(tmp_path / "deep" / "er" / "shard_0000", 10)
    assert detect_format(str(tmp_path)) == "bin"                       # found by walking the tree
    assert detect_format(str(tmp_path / "deep" / "er" / "shard_0000" / "sequence.bin")) == "bin"
    h5 = tmp_path / "file.h5"
    h5.write_bytes(b"")
    assert detect_format(str(h5)) == "h5"
    with pytest.raises(FileNotFoundError, match="No supported"):
        detect_format(str(tmp_path / "nowhere"))


# ---- stores -----------------------------------------------------------------------------------
def test_store_before_load():
    store = MmapStore()
    assert len(store) == 0 and store.keys == []
    with pytest.raises(RuntimeError, match="not loaded"):
        store.fetch(0, 1, "sequence")


def test_store_registry():
    assert isinstance(StoreFactory.create("bin"), MmapStore) and isinstance(StoreFactory.create("h5"), H5Store)
    with pytest.raises(ValueError, match="Unknown component"):
        StoreFactory.create("parquet")


def test_store_length_is_the_shortest_key(tmp_path):
    save_bin(str(tmp_path / "s"), {"sequence": [torch.arange(30, dtype=torch.int32)], "loss_mask": [torch.ones(20, dtype=torch.int32)]})
    store = MmapStore()
    store.load(str(tmp_path / "s"))
    assert len(store) == 20 and sorted(store.keys) == ["loss_mask", "sequence"]
    with pytest.raises(ValueError, match="out of bounds"):
        store.fetch(0, 21, "sequence")


def test_store_with_an_empty_key_has_length_zero():
    store = MmapStore()
    store._install({"sequence": [torch.arange(10)], "loss_mask": []})
    assert len(store) == 0
    store._install({})
    assert len(store) == 0 and store.keys == []


def test_store_fetch_across_three_shards(tmp_path):
    for i in range(3):
        _ramp(tmp_path / f"shard_{i:04d}", 10, start=10 * i)
    store = MmapStore()
    store.load(str(tmp_path))
    assert len(store) == 30
    assert store.fetch(5, 27, "sequence").tolist() == list(range(5, 27))       # first, whole middle, part of the last
    assert store.fetch(10, 20, "sequence").tolist() == list(range(10, 20))     # exactly one shard
    assert store.fetch(9, 11, "sequence").tolist() == [9, 10]
    assert store.fetch(0, 30, "sequence").tolist() == list(range(30))


def test_store_fetch_several_keys_and_empty_ranges(tmp_path):
    save_bin(str(tmp_path / "s"), {"a": [torch.arange(20, dtype=torch.int32)], "b": [torch.arange(20, 40, dtype=torch.int32)]})
    store = MmapStore()
    store.load(str(tmp_path / "s"))
    both = store.fetch(3, 6, ["a", "b"])
    assert both["a"].tolist() == [3, 4, 5] and both["b"].tolist() == [23, 24, 25]
    assert store.fetch(7, 7, "a").numel() == 0
    for begin, end in ((20, 20), (-1, 5), (0, 21), (25, 30)):
        with pytest.raises(ValueError, match="out of bounds"):
            store.fetch(begin, end, "a")


def test_store_loads_from_a_file_inside_the_shard(tmp_path):
    _ramp(tmp_path / "s", 12)
    store = MmapStore()
    store.load(str(tmp_path / "s" / "meta.json"))
    assert len(store) == 12
    with pytest.raises(FileNotFoundError):
        MmapStore().load(str(tmp_path / "empty_dir_that_does_not_exist"))


# ---- datasets ---------------------------------------------------------------------------------
def test_windows_follow_the_stride_and_the_tail_is_clamped(tmp_path):
    _ramp(tmp_path / "d", 50)
    ds = DatasetFactory.load("seq", str(tmp_path / "d"), window_size=8, stride=5)
    assert len(ds) == (50 - 1 - 8) // 5 + 1 == 9
    assert [ds.get_index(i) for i in (0, 1, 8)] == [(0, 8), (5, 13), (40, 48)]
    assert ds.get_index(100) == (41, 49)                     # past the end: the last full window
    first, second = ds[0], ds[1]
    assert first["input_ids"].tolist() == list(range(0, 8)) and first["target_ids"].tolist() == list(range(1, 9))
    assert second["input_ids"][0] == 5


def test_stride_defaults_to_the_window(tmp_path):
    _ramp(tmp_path / "d", 33)
    ds = DatasetFactory.load("seq", str(tmp_path / "d"), 8)
    assert ds.stride == 8 and len(ds) == 4 and ds[1]["input_ids"][0] == 8


def test_explicit_storage_type_skips_detection(tmp_path):
    _ramp(tmp_path / "d", 30)
    (tmp_path / "d" / "decoy.h5").write_bytes(b"")          # detection would pick h5
    ds = DatasetFactory.create("seq", 4, 4)
    ds.load(str(tmp_path / "d"), storage_type="bin")
    assert ds.count == 30 and isinstance(ds.storage, MmapStore)


def test_dataset_too_short_for_one_window(tmp_path):
    _ramp(tmp_path / "d", 8)
    ds = DatasetFactory.load("seq", str(tmp_path / "d"), 8)
    assert len(ds) == 0 and ds.count == 8
    with pytest.raises(ValueError, match="too short"):
        ds.get_index(0)


def test_unloaded_dataset():
    ds = DatasetFactory.create("sft", 4, 4)
    assert len(ds) == 0 and ds.count == 0 and ds.keys == [] and ds.required_keys == ["sequence", "loss_mask"]
    with pytest.raises(RuntimeError, match="not loaded"):
        ds[0]


def test_unknown_dataset_type():
    with pytest.raises(ValueError, match="Unknown component"):
        DatasetFactory.create("rlhf", 4, 4)
    with pytest.raises(TypeError):
        DatasetFactory.register("bad")(dict)


def test_sft_mask_is_aligned_with_the_targets(tmp_path):
    mask = torch.zeros(40, dtype=torch.int32)
    mask[10:] = 1
    save_bin(str(tmp_path / "d"), {"sequence": [torch.arange(40, dtype=torch.int32)], "loss_mask": [mask]})
    item = DatasetFactory.load("sft", str(tmp_path / "d"), 8)[1]          # window [8, 16): targets are tokens 9..16
    assert item["target_ids"].tolist() == list(range(9, 17))
    assert item["loss_mask"].tolist() == [False] + [True] * 7


def test_dataset_feeds_a_dataloader(tmp_path):
    _ramp(tmp_path / "d", 200)
    ds = DatasetFactory.load("seq", str(tmp_path / "d"), 16)
    batch = next(iter(DataLoader(ds, batch_size=4)))
    assert batch["input_ids"].shape == (4, 16) and batch["input_ids"].dtype == torch.long
    assert torch.equal(batch["target_ids"], batch["input_ids"] + 1)


# ---- sampler ----------------------------------------------------------------------------------
def test_sampler_same_seed_same_order_other_epoch_other_order():
    a = list(ResumableDistributedSampler(range(50), seed=1, num_replicas=1, rank=0))
    b = list(ResumableDistributedSampler(range(50), seed=1, num_replicas=1, rank=0))
    c = list(ResumableDistributedSampler(range(50), seed=2, num_replicas=1, rank=0))
    later = list(ResumableDistributedSampler(range(50), seed=1, start_epoch=1, num_replicas=1, rank=0))
    assert a == b and a != c and a != later and sorted(a) == sorted(later) == list(range(50))


def test_sampler_epoch_advances_after_each_pass():
    s = ResumableDistributedSampler(range(20), seed=3, num_replicas=1, rank=0)
    first, second = list(s), list(s)
    assert first != second and sorted(second) == list(range(20)) and s.epoch == 2


def test_sampler_replicas_split_the_epoch_without_overlap():
    shares = [list(ResumableDistributedSampler(range(23), seed=5, num_replicas=4, rank=r)) for r in range(4)]
    assert all(len(s) == 6 for s in shares)                              # padded to a multiple of four
    seen = [i for s in shares for i in s]
    assert set(seen) == set(range(23)) and len(seen) == 24


def test_sampler_resumes_inside_an_epoch():
    whole = list(ResumableDistributedSampler(range(40), seed=7, num_replicas=2, rank=1))
    resumed = ResumableDistributedSampler(range(40), seed=7, start_iter=6, num_replicas=2, rank=1)
    assert len(resumed) == len(whole) - 6 and list(resumed) == whole[6:]
    assert len(resumed) == len(whole)                                    # the next epoch is a full one again


def test_sampler_without_shuffle_is_ordered():
    s = ResumableDistributedSampler(range(10), shuffle=False, num_replicas=2, rank=0)
    assert list(s) == [0, 2, 4, 6, 8]


def test_sampler_set_replicas_changes_the_share():
    s = ResumableDistributedSampler(range(16), seed=1, num_replicas=4, rank=3)
    assert len(s) == 4
    s.set_replicas(2, 0)
    assert len(s) == 8 and list(s) == list(ResumableDistributedSampler(range(16), seed=1, num_replicas=2, rank=0))


def test_memory_mapped_dataset_works_in_dataloader_workers(tmp_path, method="spawn"):
    _ramp(tmp_path / "d", 1000)
    ds = DatasetFactory.load("seq", str(tmp_path / "d"), 16)
    sampler = ResumableDistributedSampler(ds, seed=1, num_replicas=1, rank=0)
    loader = DataLoader(ds, batch_size=4, sampler=sampler, num_workers=2, multiprocessing_context=method, prefetch_factor=2)
    firsts = sorted(int(x) for batch in loader for x in batch["input_ids"][:, 0])
    assert firsts == [i * 16 for i in range(len(ds))]                  # every window exactly once
