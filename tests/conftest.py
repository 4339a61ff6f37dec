import os
import sys

import pytest
import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200)")


TEST_TIMEOUT_S = 900   # no single test may hold a run longer than this (needs the pytest-timeout plugin)


def pytest_collection_modifyitems(config, items):
    if config.pluginmanager.hasplugin("timeout"):
        for item in items:
            if item.get_closest_marker("timeout") is None:
                item.add_marker(pytest.mark.timeout(TEST_TIMEOUT_S))
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(autouse=True)
def _seed():
    torch.manual_seed(3407)
    yield


@pytest.fixture(scope="session")
def tokenizer_dir(tmp_path_factory):
    """A tiny BPE tokenizer trained in-process and saved as a pretrained directory."""
    import json

    from tokenizers import Tokenizer, models, pre_tokenizers, trainers

    tk = Tokenizer(models.BPE(unk_token="<unk>"))
    tk.pre_tokenizer = pre_tokenizers.Whitespace()
    corpus = ["hello world this is a small test corpus for the tokenizer", "user assistant system question answer",
              "the quick brown fox jumps over the lazy dog"] * 30
    tk.train_from_iterator(corpus, trainers.BpeTrainer(vocab_size=300, special_tokens=["<unk>", "<bos>", "<eos>", "<pad>"]))
    d = tmp_path_factory.mktemp("tok")
    tk.save(str(d / "tokenizer.json"))
    template = "{% for m in messages %}<{{ m.role }}> {{ m.content }} <eos>\n{% endfor %}{% if add_generation_prompt %}<assistant> {% endif %}"
    (d / "tokenizer_config.json").write_text(json.dumps({
        "special_tokens": {"bos_token": "<bos>", "eos_token": "<eos>", "pad_token": "<pad>"},
        "chat_template": template}))
    return str(d)


@pytest.fixture(scope="session")
def tokenizer(tokenizer_dir):
    from khaosz_b200 import AutoTokenizer

    return AutoTokenizer.from_pretrained(tokenizer_dir)


def tiny_config(**over):
    from khaosz_b200 import AutoRegressiveLMConfig

    base = dict(vocab_size=300, dim=32, n_layers=2, norm_eps=1e-5, dim_ffn=64, tie_weight=False, max_len=64,
                rope_theta=10000.0, n_heads=4, n_kv_heads=2)
    base.update(over)
    return AutoRegressiveLMConfig(**base)


@pytest.fixture
def tiny_model():
    from khaosz_b200 import AutoRegressiveLM

    torch.manual_seed(0)
    return AutoRegressiveLM(tiny_config())


class RandomTokens(torch.utils.data.Dataset):
    def __init__(self, n=32, seq=16, vocab=300, fail_at=None):
        g = torch.Generator().manual_seed(7)
        self.data = torch.randint(0, vocab, (n, seq + 1), generator=g)
        self.fail_at, self.calls = fail_at, 0

    def __len__(self):
        return len(self.data)

    def __getitem__(self, i):
        self.calls += 1
        if self.fail_at is not None and self.calls == self.fail_at:
            raise RuntimeError("injected dataset failure")
        row = self.data[i]
        return {"input_ids": row[:-1], "target_ids": row[1:]}
