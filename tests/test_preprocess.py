import json

import pytest
import torch

from khaosz_b200.config import PipelineConfig
from khaosz_b200.data import DatasetFactory, load_bin
from khaosz_b200.preprocessing import MaskBuilderFactory, Pipeline, SectionedMaskBuilder, filter_by_length
from khaosz_b200.tokenize import ChatTemplate


def _cfg(sections, **kw):
    raw = {"input": {"sections": sections}, "mask": {"user": "mask", "assistant": "train"},
           "preprocessing": {"min_chars": 0, "max_seq_len": 64}}
    raw.update(kw)
    return PipelineConfig.from_dict(raw)


def test_tokenizer_api(tokenizer, tokenizer_dir, tmp_path):
    ids = tokenizer.encode("hello world")
    assert ids and tokenizer.decode(ids).replace(" ", "") == "helloworld"
    assert isinstance(tokenizer.encode(["hello", "world"]), list) and len(tokenizer.encode(["hello", "world"])) == 2
    assert tokenizer.bos_token == "<bos>" and isinstance(tokenizer.bos_token_id, int) and tokenizer.missing_token_id is None
    assert sorted(tokenizer.stop_ids) == sorted([tokenizer.bos_token_id, tokenizer.eos_token_id, tokenizer.pad_token_id])
    with pytest.raises(AttributeError):
        tokenizer.no_such_attr
    text = tokenizer.apply_chat_template([{"role": "user", "content": "hello"}], system_prompt="be brief", tokenize=False)
    assert text.startswith("<system> be brief") and text.endswith("<assistant> ")
    assert isinstance(tokenizer.apply_chat_template([{"role": "user", "content": "hi"}]), list)
    tokenizer.save_pretrained(str(tmp_path / "t"))
    from khaosz_b200 import AutoTokenizer

    again = AutoTokenizer.from_pretrained(str(tmp_path / "t"))
    assert again.encode("hello world") == ids and len(again) == len(tokenizer) == again.vocab_size
    with pytest.raises(FileNotFoundError):
        AutoTokenizer.from_pretrained(str(tmp_path / "missing"))
    assert ChatTemplate.from_string("{{ a }}-{{ b }}", default_variables={"a": 1}).render([], b=2) == "1-2"


def test_mask_builder_chat(tokenizer):
    b = SectionedMaskBuilder()
    cfg = _cfg([{"field": "messages", "action": "$role", "template": True}])
    item = {"messages": [{"role": "user", "content": "hello world"}, {"role": "assistant", "content": "the quick fox"}]}
    out = b.build(item, cfg, tokenizer)
    assert out["sequence"][0] == tokenizer.bos_token_id and out["loss_mask"][0] == 0 and out["domain"] == "__default__"
    user_len = len(tokenizer.encode(tokenizer.apply_chat_template([item["messages"][0]], tokenize=False,
                                                                   add_generation_prompt=False), add_special_tokens=False))
    assert sum(out["loss_mask"][: 1 + user_len]) == 0 and all(out["loss_mask"][1 + user_len:])
    all_train = b.build(item, _cfg([{"field": "messages", "action": "train", "template": True}]), tokenizer)
    assert all_train["loss_mask"].count(0) == 1  # only the BOS stays masked
    assert b.build({"messages": []}, cfg, tokenizer) is None


def test_mask_builder_instruction_and_text(tokenizer):
    b = SectionedMaskBuilder()
    cfg = _cfg([{"field": "prompt", "action": "mask"}, {"field": "response", "action": "train"}])
    out = b.build({"prompt": "hello world", "response": "the lazy dog", "src": "web"}, cfg, tokenizer)
    n_prompt = len(tokenizer.encode("hello world"))
    assert out["loss_mask"][:n_prompt] == [0] * n_prompt and all(out["loss_mask"][n_prompt:])
    text_cfg = _cfg([{"field": "text", "action": "train"}], preprocessing={"min_chars": 5, "max_seq_len": 4},
                    output={"domain_key": "src"})
    out = b.build({"text": "the quick brown fox jumps", "src": "web"}, text_cfg, tokenizer)
    assert "loss_mask" not in out and len(out["sequence"]) == 4 and out["domain"] == "web"
    assert b.build({"text": "hi"}, text_cfg, tokenizer) is None  # below min_chars
    assert MaskBuilderFactory.is_registered("sectioned") and filter_by_length("x" * 60) and not filter_by_length("x")


def test_pipeline_outputs(tokenizer_dir, tmp_path):
    src = tmp_path / "in.jsonl"
    rows = [{"text": "the quick brown fox jumps over the lazy dog " * 3, "kind": "a"},
            {"text": "hello world this is a test corpus " * 3, "kind": "b"},
            {"text": "", "kind": "a"}]
    src.write_text("\n".join(json.dumps(r) for r in rows) + "\n\n")
    cfg = _cfg([{"field": "text", "action": "train"}])
    assert Pipeline(cfg, [str(src)], str(tmp_path / "out"), tokenizer_dir).run() == 2
    meta = json.loads((tmp_path / "out" / "__default__" / "shard_0000" / "meta.json").read_text())
    assert meta["sequence"]["dtype"] == "int32" and "loss_mask" not in meta
    ds = DatasetFactory.load("seq", str(tmp_path / "out"), 8)
    assert len(ds) > 0
    # domains, late loss_mask back-fill, dtype override, several shards
    chat = tmp_path / "chat.jsonl"
    chat.write_text("\n".join(json.dumps(r) for r in [
        {"prompt": "", "response": "the lazy dog", "kind": "a"},
        {"prompt": "hello world", "response": "the quick fox", "kind": "a"},
        {"prompt": "hello", "response": "dog", "kind": "b"}]))
    cfg2 = _cfg([{"field": "prompt", "action": "mask"}, {"field": "response", "action": "train"}],
                output={"domain_key": "kind", "dtype": {"loss_mask": "bool", "sequence": "int64"},
                        "max_tokens_per_shard": 8})
    Pipeline(cfg2, [str(chat)], str(tmp_path / "out2"), tokenizer_dir).run()
    a0 = load_bin(str(tmp_path / "out2" / "a" / "shard_0000"))
    assert a0["sequence"][0].dtype == torch.int64 and a0["loss_mask"][0].dtype == torch.bool
    assert a0["loss_mask"][0].numel() == a0["sequence"][0].numel()
    assert (tmp_path / "out2" / "b").exists()
