"""The HDF5 side of the token storage (``save_h5`` / ``load_h5`` / ``H5Store`` / the preprocessing
pipeline's ``h5`` output), run through ``h5py`` when the host has it and through the stand-in of
``tests/fake_h5py.py`` otherwise (reference: ``astrai/dataset/storage.py:36-69,231-236``)."""
import json
import sys

import pytest
import torch

import fake_h5py


@pytest.fixture()
def h5(monkeypatch):
    try:
        import h5py  # noqa: F401

        yield "real"
    except ImportError:
        assert fake_h5py.install()
        yield "stand-in"
        sys.modules.pop("h5py", None)


def test_save_and_load_h5_round_trip(tmp_path, h5):
    from khaosz_b200.data.storage import detect_format, load_h5, save_h5

    group = {"sequence": [torch.arange(10, dtype=torch.int32), torch.arange(10, 25, dtype=torch.int32)],
             "loss_mask": [torch.ones(25, dtype=torch.bool)]}
    save_h5(str(tmp_path), "data_0000", group)
    assert (tmp_path / "data_0000.h5").exists() and detect_format(str(tmp_path)) == "h5"
    back = load_h5(str(tmp_path))
    assert set(back) == {"sequence", "loss_mask"} and len(back["sequence"]) == 2
    assert torch.equal(back["sequence"][1], group["sequence"][1]) and back["sequence"][0].dtype == torch.int32
    assert back["loss_mask"][0].dtype == torch.bool and back["sequence"][0].is_shared()


def test_h5_store_fetches_across_segments_and_files(tmp_path, h5):
    from khaosz_b200.data import DatasetFactory
    from khaosz_b200.data.storage import H5Store, StoreFactory, save_h5

    save_h5(str(tmp_path), "a", {"sequence": [torch.arange(0, 40), torch.arange(40, 100)]})
    save_h5(str(tmp_path), "b", {"sequence": [torch.arange(100, 130)]})
    store = StoreFactory.create("h5")
    assert isinstance(store, H5Store)
    with pytest.raises(RuntimeError, match="not loaded"):
        store.fetch(0, 1, "sequence")
    store.load(str(tmp_path))
    assert len(store) == 130 and store.keys == ["sequence"]
    assert store.fetch(35, 45, "sequence").tolist() == list(range(35, 45))      # crosses a segment boundary
    assert store.fetch(95, 105, "sequence").tolist() == list(range(95, 105))    # crosses a file boundary
    with pytest.raises(ValueError, match="out of bounds"):
        store.fetch(0, 131, "sequence")
    ds = DatasetFactory.load("seq", str(tmp_path), window_size=16)            # format detected from the files
    assert ds.count == 130 and len(ds) == (130 - 1 - 16) // 16 + 1
    item = ds[1]
    assert item["input_ids"].tolist() == list(range(16, 32)) and item["target_ids"].tolist() == list(range(17, 33))


def test_pipeline_writes_h5_shards(tmp_path, h5, tokenizer_dir, tokenizer):
    from khaosz_b200.config import PipelineConfig
    from khaosz_b200.data.storage import load_h5
    from khaosz_b200.preprocessing import Pipeline

    docs = ["hello world this is a small test corpus " * (3 + i) for i in range(5)]
    src = tmp_path / "in.jsonl"
    src.write_text("\n".join(json.dumps({"text": d}) for d in docs))
    cfg = PipelineConfig.from_dict({"version": 1, "input": {"sections": [{"field": "text", "action": "train"}]},
                                    "output": {"storage_format": "h5", "max_tokens_per_shard": 60}})
    assert Pipeline(cfg, [str(src)], str(tmp_path / "out"), tokenizer_dir).run() == 5
    files = sorted((tmp_path / "out" / "__default__").glob("*.h5"))
    assert len(files) >= 2 and files[0].name == "data_0000.h5"
    back = load_h5(str(tmp_path / "out"))
    total = sum(len(tokenizer.encode(d)) for d in docs)
    assert sum(t.numel() for t in back["sequence"]) >= total and back["sequence"][0].dtype == torch.int32
