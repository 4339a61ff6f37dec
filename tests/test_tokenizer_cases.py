"""Case-by-case behaviour of ``AutoTokenizer`` and ``ChatTemplate``
(reference: ``astrai/tokenize/tokenizer.py:35-180``, ``astrai/tokenize/chat_template.py:8-74``)."""
import json

import pytest

from khaosz_b200 import AutoTokenizer
from khaosz_b200.tokenize import ChatTemplate


# ---- encode / decode --------------------------------------------------------------------------
def test_encode_text_gives_ids_and_decode_gives_the_words_back(tokenizer):
    ids = tokenizer.encode("hello world")
    assert ids and all(isinstance(i, int) and 0 <= i < len(tokenizer) for i in ids)
    assert tokenizer.decode(ids).split() == ["hello", "world"]


def test_encode_a_list_gives_one_row_per_text(tokenizer):
    rows = tokenizer.encode(["hello world", "the lazy dog", ""])
    assert len(rows) == 3 and rows[0] == tokenizer.encode("hello world") and rows[2] == []


def test_encode_can_return_token_strings(tokenizer):
    pieces = tokenizer.encode("hello world", out_ids=False)
    assert all(isinstance(p, str) for p in pieces) and "".join(pieces) == "helloworld"
    assert [tokenizer._tokenizer.token_to_id(p) for p in pieces] == tokenizer.encode("hello world")


def test_encode_pretokenized_input(tokenizer):
    rows = tokenizer.encode([["hello", "world"], ["the", "lazy", "dog"]], is_pretokenized=True)   # a batch of word lists
    assert rows == [tokenizer.encode("hello world"), tokenizer.encode("the lazy dog")]


def test_decode_can_keep_special_tokens(tokenizer):
    ids = [tokenizer.bos_token_id] + tokenizer.encode("hello") + [tokenizer.eos_token_id]
    assert "<bos>" not in tokenizer.decode(ids) and "<eos>" not in tokenizer.decode(ids)
    kept = tokenizer.decode(ids, skip_special_tokens=False)
    assert "<bos>" in kept and "<eos>" in kept


def test_vocabulary_size(tokenizer):
    assert len(tokenizer) == tokenizer.vocab_size > 4
    assert len(AutoTokenizer()) == 0


# ---- special tokens ---------------------------------------------------------------------------
def test_special_tokens_are_attributes_with_ids(tokenizer):
    assert (tokenizer.bos_token, tokenizer.eos_token, tokenizer.pad_token) == ("<bos>", "<eos>", "<pad>")
    ids = (tokenizer.bos_token_id, tokenizer.eos_token_id, tokenizer.pad_token_id)
    assert all(isinstance(i, int) for i in ids) and len(set(ids)) == 3
    assert tokenizer.decode([tokenizer.eos_token_id], skip_special_tokens=False) == "<eos>"


def test_unknown_special_tokens(tokenizer):
    assert tokenizer.sep_token_id is None                  # `*_id` of a token that is not configured
    with pytest.raises(AttributeError):
        tokenizer.sep_token
    with pytest.raises(AttributeError):
        tokenizer._private


def test_stop_ids_are_all_special_tokens(tokenizer):
    assert sorted(tokenizer.stop_ids) == sorted([tokenizer.bos_token_id, tokenizer.eos_token_id, tokenizer.pad_token_id])
    assert AutoTokenizer().stop_ids == []


def test_unloaded_tokenizer_raises_clearly():
    empty = AutoTokenizer(special_token_map={"bos_token": "<bos>"})
    assert empty.bos_token == "<bos>"
    with pytest.raises(RuntimeError, match="not initialized"):
        empty.encode("hello")
    with pytest.raises(RuntimeError, match="not loaded"):
        empty.bos_token_id
    with pytest.raises(RuntimeError, match="not initialized"):
        empty.save_pretrained("/tmp/never_written")


# ---- files ------------------------------------------------------------------------------------
def test_save_and_load_keep_vocabulary_special_tokens_and_template(tokenizer, tmp_path):
    tokenizer.save_pretrained(str(tmp_path / "tok"))
    assert sorted(p.name for p in (tmp_path / "tok").iterdir()) == ["tokenizer.json", "tokenizer_config.json"]
    cfg = json.loads((tmp_path / "tok" / "tokenizer_config.json").read_text())
    assert cfg["special_tokens"]["eos_token"] == "<eos>" and "chat_template" in cfg
    back = AutoTokenizer.from_pretrained(str(tmp_path / "tok"))
    text = "the quick brown fox"
    assert back.encode(text) == tokenizer.encode(text) and back.stop_ids == tokenizer.stop_ids
    messages = [{"role": "user", "content": "hello"}]
    assert back.apply_chat_template(messages, tokenize=False) == tokenizer.apply_chat_template(messages, tokenize=False)


def test_loading_needs_a_tokenizer_file(tmp_path):
    with pytest.raises(FileNotFoundError, match="tokenizer.json"):
        AutoTokenizer.from_pretrained(str(tmp_path))


def test_tokenizer_without_a_config_file_still_loads(tokenizer_dir, tmp_path):
    import shutil

    shutil.copy(f"{tokenizer_dir}/tokenizer.json", tmp_path / "tokenizer.json")
    bare = AutoTokenizer.from_pretrained(str(tmp_path))
    assert bare.encode("hello world") and bare.stop_ids == []
    with pytest.raises(RuntimeError, match="Chat template not set"):
        bare.apply_chat_template([{"role": "user", "content": "x"}])


def test_custom_tokenizer_classes_can_be_registered():
    class Mine:
        pass

    AutoTokenizer.register_tokenizer("mine", Mine)
    assert AutoTokenizer.TOKENIZER_CLASSES["mine"] is Mine
    del AutoTokenizer.TOKENIZER_CLASSES["mine"]


# ---- chat template ----------------------------------------------------------------------------
def test_chat_template_renders_roles_in_order_with_a_generation_prompt(tokenizer):
    messages = [{"role": "user", "content": "hello"}, {"role": "assistant", "content": "world"}, {"role": "user", "content": "fox"}]
    text = tokenizer.apply_chat_template(messages, tokenize=False)
    assert text.index("<user> hello") < text.index("<assistant> world") < text.index("<user> fox")
    assert text.endswith("<assistant> ")
    closed = tokenizer.apply_chat_template(messages, tokenize=False, add_generation_prompt=False)
    assert not closed.endswith("<assistant> ") and text.startswith(closed)


def test_chat_template_system_prompt_comes_first(tokenizer):
    text = tokenizer.apply_chat_template([{"role": "user", "content": "hello"}], system_prompt="be brief", tokenize=False)
    assert text.startswith("<system> be brief") and "<user> hello" in text
    plain = tokenizer.apply_chat_template([{"role": "user", "content": "hello"}], system_prompt="", tokenize=False)
    assert "<system>" not in plain


def test_chat_template_tokenizes_by_default(tokenizer):
    messages = [{"role": "user", "content": "hello"}]
    ids = tokenizer.apply_chat_template(messages)
    assert ids == tokenizer.encode(tokenizer.apply_chat_template(messages, tokenize=False))


def test_chat_template_can_be_replaced(tokenizer_dir):
    tok = AutoTokenizer.from_pretrained(tokenizer_dir)
    tok.set_chat_template("{% for m in messages %}[{{ m.role }}:{{ m.content }}]{% endfor %}")
    assert tok.apply_chat_template([{"role": "user", "content": "hi"}], tokenize=False) == "[user:hi]"
    tok.set_chat_template(ChatTemplate.from_string("{{ messages | length }} turns"))
    assert tok.apply_chat_template([{"role": "user", "content": "a"}] * 3, tokenize=False) == "3 turns"
    with pytest.raises(ValueError, match="Invalid template type"):
        tok.set_chat_template(42)


def test_chat_template_variables():
    tpl = ChatTemplate.from_string("{{ greeting }}, {{ name }}!{% if system_prompt %} ({{ system_prompt }}){% endif %}",
                                   default_variables={"greeting": "hello"})
    assert tpl.render([], name="fox") == "hello, fox!"
    assert tpl.render([], name="fox", greeting="bye") == "bye, fox!"                 # a call-time value wins
    assert tpl.render([], system_prompt="short", name="dog") == "hello, dog! (short)"
    assert ChatTemplate(name="n", template_str="x", description="d").template_str == "x"
