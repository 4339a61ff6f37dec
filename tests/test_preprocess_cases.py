"""Case-by-case behaviour of the preprocessing configs, the sectioned mask builder and the pipeline
(the behaviours the reference pins in ``tests/data/test_preprocess.py``)."""
import json

import pytest
import torch

from khaosz_b200.config import PipelineConfig
from khaosz_b200.config.pipeline_config import InputConfig, OutputConfig, ProcessingConfig
from khaosz_b200.data import DatasetFactory, load_bin
from khaosz_b200.preprocessing import MaskBuilderFactory, Pipeline, SectionedMaskBuilder, filter_by_length

CHAT = [{"field": "messages", "action": "$role", "template": True}]
INSTRUCT = [{"field": "prompt", "action": "mask"}, {"field": "response", "action": "train"}]
TEXT = [{"field": "text", "action": "train"}]
TALK = {"messages": [{"role": "user", "content": "hello world"}, {"role": "assistant", "content": "the quick fox"},
                     {"role": "user", "content": "this is a test"}, {"role": "assistant", "content": "the lazy dog"}]}


def _cfg(sections, mask=None, **kw):
    raw = {"input": {"sections": sections}, "mask": {"user": "mask", "assistant": "train"} if mask is None else mask,
           "preprocessing": {"min_chars": 0, "max_seq_len": 128}}
    raw.update(kw)
    return PipelineConfig.from_dict(raw)


def _message_len(tokenizer, message):
    text = tokenizer.apply_chat_template([message], tokenize=False, add_generation_prompt=False)
    return len(tokenizer.encode(text, add_special_tokens=False))


# ---- configs ---------------------------------------------------------------------------------
def test_config_defaults():
    cfg = PipelineConfig()
    assert cfg.version == 1 and cfg.mask == {} and cfg.mask_default == "mask"
    assert cfg.input.sections is None and list(cfg.input.iter_sections()) == []
    assert (cfg.preprocessing.max_seq_len, cfg.preprocessing.min_chars, cfg.preprocessing.max_chars,
            cfg.preprocessing.max_items) == (2048, 50, 2_000_000, None)
    assert (cfg.output.domain_key, cfg.output.storage_format, cfg.output.max_tokens_per_shard, cfg.output.dtype) == \
        (None, "bin", 100_000_000, {})
    assert cfg.output.dtype_of("sequence") == "int32"


def test_config_from_dict_builds_nested_sections():
    cfg = PipelineConfig.from_dict({"input": {"sections": CHAT}, "mask": {"assistant": "train"}, "mask_default": "mask",
                                    "preprocessing": {"max_seq_len": 99}, "output": {"domain_key": "src", "dtype": {"loss_mask": "bool"}}})
    assert isinstance(cfg.input, InputConfig) and isinstance(cfg.preprocessing, ProcessingConfig)
    assert isinstance(cfg.output, OutputConfig)
    assert cfg.input.sections[0]["field"] == "messages" and cfg.preprocessing.max_seq_len == 99
    assert cfg.preprocessing.min_chars == 50                       # untouched fields keep their defaults
    assert cfg.output.dtype_of("loss_mask") == "bool" and cfg.output.dtype_of("sequence") == "int32"
    assert cfg.action_for_role("assistant") == "train" and cfg.action_for_role("tool") == "mask"


def test_config_dict_and_json_round_trip(tmp_path):
    cfg = _cfg(INSTRUCT, output={"domain_key": "kind", "max_tokens_per_shard": 77})
    again = PipelineConfig.from_dict(cfg.to_dict())
    assert again.to_dict() == cfg.to_dict()
    path = tmp_path / "pipeline.json"
    cfg.to_json(str(path))
    loaded = PipelineConfig.from_json(str(path))
    assert loaded.to_dict() == cfg.to_dict() and loaded.output.max_tokens_per_shard == 77
    assert json.loads(path.read_text())["input"]["sections"][1]["action"] == "train"


def test_processing_limits():
    limits = ProcessingConfig(min_chars=3, max_chars=5)
    assert limits.keep_text("abc") and limits.keep_text("abcde")
    assert not limits.keep_text("ab") and not limits.keep_text("abcdef")
    assert filter_by_length("x" * 50) and not filter_by_length("x" * 49) and not filter_by_length("x" * 11, 1, 10)


# ---- chat -----------------------------------------------------------------------------------
def test_chat_trains_assistant_turns_only(tokenizer):
    out = SectionedMaskBuilder().build(TALK, _cfg(CHAT), tokenizer)
    lens = [_message_len(tokenizer, m) for m in TALK["messages"]]
    assert len(out["sequence"]) == 1 + sum(lens) == len(out["loss_mask"])
    pos, want = 1, [0]
    for n, msg in zip(lens, TALK["messages"]):
        want += [int(msg["role"] == "assistant")] * n
        pos += n
    assert out["loss_mask"] == want and out["sequence"][0] == tokenizer.bos_token_id


def test_chat_roles_missing_from_the_mask_use_the_default(tokenizer):
    item = {"messages": [{"role": "tool", "content": "hello"}, {"role": "assistant", "content": "world"}]}
    masked = SectionedMaskBuilder().build(item, _cfg(CHAT, mask={"assistant": "train"}), tokenizer)
    first = _message_len(tokenizer, item["messages"][0])
    assert sum(masked["loss_mask"][:1 + first]) == 0 and all(masked["loss_mask"][1 + first:])
    trained = SectionedMaskBuilder().build(item, _cfg(CHAT, mask={"assistant": "mask"}, mask_default="train"), tokenizer)
    assert all(trained["loss_mask"][1:1 + first]) and sum(trained["loss_mask"][1 + first:]) == 0


def test_chat_everything_masked_keeps_an_all_zero_mask(tokenizer):
    out = SectionedMaskBuilder().build(TALK, _cfg(CHAT, mask={"user": "mask", "assistant": "mask"}), tokenizer)
    assert out is not None and sum(out["loss_mask"]) == 0 and len(out["loss_mask"]) == len(out["sequence"])


def test_chat_everything_trained_masks_only_the_bos(tokenizer):
    out = SectionedMaskBuilder().build(TALK, _cfg(CHAT, mask={"user": "train", "assistant": "train"}), tokenizer)
    assert out["loss_mask"][0] == 0 and all(out["loss_mask"][1:])


@pytest.mark.parametrize("item", [{"messages": []}, {"messages": None}, {}, {"messages": "not a list"}])
def test_chat_without_messages_is_skipped(tokenizer, item):
    assert SectionedMaskBuilder().build(item, _cfg(CHAT), tokenizer) is None


def test_domain_comes_from_the_configured_key(tokenizer):
    b = SectionedMaskBuilder()
    cfg = _cfg(CHAT, output={"domain_key": "source"})
    assert b.build({**TALK, "source": "forum"}, cfg, tokenizer)["domain"] == "forum"
    assert b.build(TALK, cfg, tokenizer)["domain"] == "__default__"              # key absent
    assert b.build({**TALK, "source": 7}, cfg, tokenizer)["domain"] == "__default__"   # not a string
    assert b.build({**TALK, "source": "forum"}, _cfg(CHAT), tokenizer)["domain"] == "__default__"   # no key configured


def test_chat_is_cut_to_max_seq_len(tokenizer):
    out = SectionedMaskBuilder().build(TALK, _cfg(CHAT, preprocessing={"min_chars": 0, "max_seq_len": 7}), tokenizer)
    assert len(out["sequence"]) == 7 == len(out["loss_mask"])


# ---- instruction ------------------------------------------------------------------------------
def test_instruction_masks_the_prompt_and_trains_the_response(tokenizer):
    item = {"prompt": "hello world", "response": "the lazy dog"}
    out = SectionedMaskBuilder().build(item, _cfg(INSTRUCT), tokenizer)
    n_prompt = len(tokenizer.encode("hello world"))
    n_resp = len(tokenizer.encode("the lazy dog", add_special_tokens=False))
    assert len(out["sequence"]) == n_prompt + n_resp
    assert out["loss_mask"] == [0] * n_prompt + [1] * n_resp
    assert out["sequence"][n_prompt:] == tokenizer.encode("the lazy dog", add_special_tokens=False)


def test_instruction_can_train_on_the_prompt_too(tokenizer):
    both = [{"field": "prompt", "action": "train"}, {"field": "response", "action": "train"}]
    out = SectionedMaskBuilder().build({"prompt": "hello world", "response": "the lazy dog"}, _cfg(both), tokenizer)
    assert "loss_mask" not in out            # nothing masked: the key is left out
    assert len(out["sequence"]) == len(tokenizer.encode("hello world")) + len(tokenizer.encode("the lazy dog", add_special_tokens=False))


def test_instruction_with_an_empty_prompt_still_trains_the_response(tokenizer):
    out = SectionedMaskBuilder().build({"prompt": "   ", "response": "the lazy dog"}, _cfg(INSTRUCT), tokenizer)
    assert out is not None and "loss_mask" not in out
    assert SectionedMaskBuilder().build({"prompt": "", "response": ""}, _cfg(INSTRUCT), tokenizer) is None


def test_instruction_ignores_the_character_limits(tokenizer):
    """``min_chars`` filters plain-text records only: a short answer is still a sample."""
    cfg = _cfg(INSTRUCT, preprocessing={"min_chars": 500, "max_seq_len": 64})
    assert SectionedMaskBuilder().build({"prompt": "hello", "response": "dog"}, cfg, tokenizer) is not None


# ---- plain text -------------------------------------------------------------------------------
def test_text_has_no_loss_mask(tokenizer):
    out = SectionedMaskBuilder().build({"text": "the quick brown fox"}, _cfg(TEXT), tokenizer)
    assert set(out) == {"sequence", "domain"} and out["sequence"] == tokenizer.encode("the quick brown fox")


@pytest.mark.parametrize("text", ["", "   ", None])
def test_text_empty_is_skipped(tokenizer, text):
    item = {} if text is None else {"text": text}
    assert SectionedMaskBuilder().build(item, _cfg(TEXT), tokenizer) is None


def test_text_length_limits(tokenizer):
    b = SectionedMaskBuilder()
    cfg = _cfg(TEXT, preprocessing={"min_chars": 10, "max_chars": 30, "max_seq_len": 64})
    assert b.build({"text": "too short"}, cfg, tokenizer) is None
    assert b.build({"text": "the quick brown fox"}, cfg, tokenizer) is not None
    assert b.build({"text": "the quick brown fox jumps over the lazy dog"}, cfg, tokenizer) is None


def test_text_is_cut_to_max_seq_len(tokenizer):
    cfg = _cfg(TEXT, preprocessing={"min_chars": 0, "max_seq_len": 3})
    out = SectionedMaskBuilder().build({"text": "the quick brown fox jumps over the lazy dog"}, cfg, tokenizer)
    assert out["sequence"] == tokenizer.encode("the quick brown fox jumps over the lazy dog")[:3]


def test_no_sections_builds_nothing(tokenizer):
    assert SectionedMaskBuilder().build({"text": "hello world"}, PipelineConfig(), tokenizer) is None


def test_mask_builder_registry():
    assert "sectioned" in MaskBuilderFactory.list_registered()
    assert isinstance(MaskBuilderFactory.create("sectioned"), SectionedMaskBuilder)
    with pytest.raises(ValueError, match="Unknown component"):
        MaskBuilderFactory.create("no_such_builder")
    with pytest.raises(TypeError):
        MaskBuilderFactory.register("bad")(dict)


# ---- whole pipeline -----------------------------------------------------------------------------
def _write(path, rows):
    path.write_text("\n".join(json.dumps(r) for r in rows) + "\n")
    return str(path)


def test_pipeline_chat_writes_sequence_and_mask_of_equal_length(tokenizer_dir, tokenizer, tmp_path):
    rows = [TALK, {"messages": [{"role": "user", "content": "hello"}, {"role": "assistant", "content": "world"}]}, {"messages": []}]
    n = Pipeline(_cfg(CHAT), [_write(tmp_path / "chat.jsonl", rows)], str(tmp_path / "out"), tokenizer_dir).run()
    assert n == 2
    shard = tmp_path / "out" / "__default__" / "shard_0000"
    meta = json.loads((shard / "meta.json").read_text())
    assert set(meta) == {"sequence", "loss_mask"} and meta["sequence"]["dtype"] == meta["loss_mask"]["dtype"] == "int32"
    data = load_bin(str(shard))
    seq, mask = torch.cat(data["sequence"]), torch.cat(data["loss_mask"])
    assert seq.numel() == mask.numel() and 0 < int(mask.sum()) < mask.numel()
    assert int((seq == tokenizer.bos_token_id).sum()) == 2            # one BOS per conversation
    ds = DatasetFactory.load("sft", str(tmp_path / "out"), 8)
    item = ds[0]
    assert set(item) == {"input_ids", "target_ids", "loss_mask"} and item["loss_mask"].dtype == torch.bool


def test_pipeline_text_writes_no_mask(tokenizer_dir, tmp_path):
    rows = [{"text": "the quick brown fox jumps over the lazy dog " * 2}, {"text": "hello world this is a test " * 2}]
    assert Pipeline(_cfg(TEXT), [_write(tmp_path / "t.jsonl", rows)], str(tmp_path / "out"), tokenizer_dir).run() == 2
    shard = tmp_path / "out" / "__default__" / "shard_0000"
    assert sorted(p.name for p in shard.iterdir()) == ["meta.json", "sequence.bin"]
    assert load_bin(str(shard))["sequence"][0].dtype == torch.int32


def test_pipeline_instruction_splits_domains(tokenizer_dir, tmp_path):
    rows = [{"prompt": "hello world", "response": "the lazy dog", "kind": "qa"},
            {"prompt": "this is a test", "response": "the quick fox", "kind": "qa"},
            {"prompt": "hello", "response": "dog", "kind": "chitchat"},
            {"prompt": "hello", "response": "fox"}]
    cfg = _cfg(INSTRUCT, output={"domain_key": "kind"})
    assert Pipeline(cfg, [_write(tmp_path / "i.jsonl", rows)], str(tmp_path / "out"), tokenizer_dir).run() == 4
    assert sorted(p.name for p in (tmp_path / "out").iterdir()) == ["__default__", "chitchat", "qa"]
    qa = load_bin(str(tmp_path / "out" / "qa" / "shard_0000"))
    assert torch.cat(qa["sequence"]).numel() == torch.cat(qa["loss_mask"]).numel()


def test_pipeline_dtype_override_and_max_items(tokenizer_dir, tmp_path):
    rows = [{"prompt": "hello world", "response": "the lazy dog"}] * 5
    cfg = _cfg(INSTRUCT, output={"dtype": {"sequence": "int64", "loss_mask": "bool"}},
               preprocessing={"min_chars": 0, "max_seq_len": 64, "max_items": 3})
    assert Pipeline(cfg, [_write(tmp_path / "i.jsonl", rows)], str(tmp_path / "out"), tokenizer_dir).run() == 3
    meta = json.loads((tmp_path / "out" / "__default__" / "shard_0000" / "meta.json").read_text())
    assert meta["sequence"]["dtype"] == "int64" and meta["loss_mask"]["dtype"] == "bool"


def test_pipeline_starts_a_new_shard_at_the_token_limit(tokenizer_dir, tokenizer, tmp_path):
    rows = [{"text": "the quick brown fox jumps over the lazy dog"}] * 6
    cfg = _cfg(TEXT, output={"max_tokens_per_shard": 20})
    Pipeline(cfg, [_write(tmp_path / "t.jsonl", rows)], str(tmp_path / "out"), tokenizer_dir).run()
    shards = sorted(p.name for p in (tmp_path / "out" / "__default__").iterdir())
    assert len(shards) >= 2 and shards[0] == "shard_0000" and shards[1] == "shard_0001"
    total = sum(torch.cat(load_bin(str(tmp_path / "out" / "__default__" / s))["sequence"]).numel() for s in shards)
    assert total == 6 * len(tokenizer.encode("the quick brown fox jumps over the lazy dog"))     # nothing lost between shards
    ds = DatasetFactory.load("seq", str(tmp_path / "out"), 8)          # the shards read back as one stream
    assert ds.count == total


def test_pipeline_reads_several_files_and_skips_bad_lines(tokenizer_dir, tmp_path):
    a = _write(tmp_path / "a.jsonl", [{"text": "the quick brown fox jumps"}])
    b = tmp_path / "b.jsonl"
    b.write_text(json.dumps({"text": "hello world this is a test"}) + "\n\nnot json at all\n[1, 2, 3]\n42\n"
                 + json.dumps({"text": "the lazy dog"}) + "\n")
    job = Pipeline(_cfg(TEXT), [a, str(b)], str(tmp_path / "out"), tokenizer_dir)
    assert job.run() == 3 and job.skipped_lines == 3          # damaged text, a list and a number are not records


def test_malformed_turns_are_dropped_and_the_dialogue_kept(tokenizer):
    good = SectionedMaskBuilder().build(TALK, _cfg(CHAT), tokenizer)
    noisy = {"messages": [TALK["messages"][0], "not a turn", None, *TALK["messages"][1:]]}
    assert SectionedMaskBuilder().build(noisy, _cfg(CHAT), tokenizer) == good
    assert SectionedMaskBuilder().build({"messages": ["only junk", 7]}, _cfg(CHAT), tokenizer) is None
    assert SectionedMaskBuilder().build({"text": 12345}, _cfg(TEXT), tokenizer)["sequence"] == tokenizer.encode("12345")
