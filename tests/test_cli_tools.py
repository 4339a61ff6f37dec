"""Smoke tests of the command-line tools on CPU with a tiny saved model and tokenizer."""
import json
import shutil

import pytest
import torch

from khaosz_b200 import AutoRegressiveLM, AutoRegressiveLMConfig


@pytest.fixture
def param_dir(tmp_path, tokenizer_dir, tokenizer):
    d = tmp_path / "params"
    shutil.copytree(tokenizer_dir, d)
    cfg = AutoRegressiveLMConfig(vocab_size=len(tokenizer), dim=32, n_layers=2, norm_eps=1e-5, dim_ffn=64, tie_weight=False,
                                 max_len=64, rope_theta=1e4, n_heads=4, n_kv_heads=2)
    torch.manual_seed(0)
    AutoRegressiveLM(cfg).save_pretrained(str(d))
    return d


def test_generate_cli_writes_one_response_per_question(param_dir, tmp_path):
    from khaosz_b200.cli import generate

    src, dst = tmp_path / "q.jsonl", tmp_path / "a.jsonl"
    src.write_text("\n".join(json.dumps({"question": q}) for q in ("hello world", "the quick brown fox")) + "\n")
    a = generate.parse_args(["--param_path", str(param_dir), "--input_json_file", str(src), "--output_json_file", str(dst),
                             "--max_tokens", "4", "--batch_size", "2", "--device", "cpu", "--top_k", "1"])
    generate.run(a)
    rows = [json.loads(l) for l in dst.read_text().splitlines() if l.strip()]
    assert len(rows) == 2 and all("response" in r and "question" in r for r in rows)


def test_perplexity_cli_reports_finite_values(param_dir, tmp_path):
    from khaosz_b200.cli import perplexity

    src, dst = tmp_path / "t.jsonl", tmp_path / "p.jsonl"
    src.write_text("\n".join(json.dumps({"text": t}) for t in ("hello world this is a test", "the lazy dog")) + "\n")
    a = perplexity.parse_args(["--param_path", str(param_dir), "--input_file", str(src), "--output_file", str(dst),
                               "--batch_size", "2", "--device", "cpu"])
    perplexity.run(a)
    rows = [json.loads(l) for l in dst.read_text().splitlines() if l.strip()]
    assert len(rows) == 2
    vals = [v for r in rows for v in r.values() if isinstance(v, float)]
    assert vals and all(v == v and v > 0 for v in vals)


def test_cli_reference_lists_every_flag():
    """docs/cli.md is generated from the parsers; a flag added to a tool has to show up there."""
    import contextlib
    import importlib
    import io
    import re
    from pathlib import Path

    text = (Path(__file__).resolve().parent.parent / "docs" / "cli.md").read_text()
    sections = {m.group(1): m.end() for m in re.finditer(r"^## `python -m khaosz_b200\.cli\.(\w+)`", text, re.M)}
    assert {"train", "server", "generate", "perplexity", "evaluate_mmlu", "preprocess", "benchmark", "demo",
            "kernel_bench", "comm_bench"} <= set(sections)
    order = sorted(sections.values()) + [len(text)]
    for tool, start in sections.items():
        body = text[start:order[order.index(start) + 1]]
        mod = importlib.import_module(f"khaosz_b200.cli.{tool}")
        buf = io.StringIO()
        with contextlib.redirect_stdout(buf), contextlib.redirect_stderr(buf):
            try:
                (getattr(mod, "parse_args", None) or mod.main)(["--help"])
            except SystemExit:
                pass
        flags = set(re.findall(r"(?<![\w-])--[a-z][\w-]*", buf.getvalue()))
        missing = sorted(f for f in flags if f not in body)
        assert not missing, f"docs/cli.md section of {tool} lacks {missing}"


def _mmlu_dir(tmp_path):
    root = tmp_path / "mmlu"
    rows = [["the quick brown fox is", "A) lazy", "B) quick", "C) a dog", "D) hello", "B"],
            ["hello world is a", "test", "corpus", "question", "answer", "A"],
            ["this is a small", "world", "dog", "test", "fox", "C"]]
    for split, subset in (("dev", rows[:2]), ("test", rows)):
        (root / split).mkdir(parents=True)
        for subject in ("toy_logic", "toy_words"):
            with open(root / split / f"{subject}_{split}.csv", "w", encoding="utf-8") as fh:
                fh.write("question,A,B,C,D,answer\n")            # a header line is tolerated
                for r in subset:
                    fh.write(",".join(r) + "\n")
    return root


def test_mmlu_tool_scores_every_question_and_writes_a_summary(param_dir, tmp_path):
    from khaosz_b200.cli import evaluate_mmlu as tool

    data = _mmlu_dir(tmp_path)
    rows = tool.load_csv(str(data / "test" / "toy_logic_test.csv"))
    assert len(rows) == 3 and rows[0]["B"] == "quick" and rows[0]["answer"] == "B" and rows[1]["A"] == "test"
    prompt = tool.build_prompt(rows[2]["question"], rows[2], "toy logic", 1, rows[:2])
    assert prompt.startswith("The following are multiple choice questions (with answers) about toy logic.")
    assert prompt.count("Answer:") == 2 and prompt.endswith("Answer:") and "Answer: B\n" in prompt
    assert tool.build_prompt(rows[2]["question"], rows[2], "toy logic", 0, rows[:2]).count("Question:") == 1
    out = tmp_path / "mmlu.json"
    summary = tool.run(tool.parse_args(["--param_path", str(param_dir), "--data_dir", str(data), "--n_shot", "2",
                                        "--device", "cpu", "--dtype", "float32", "--output", str(out)]))
    assert summary["total"] == 6 and set(summary["subjects"]) == {"toy_logic", "toy_words"}
    assert 0.0 <= summary["average"] <= 1.0 and summary["correct"] == sum(s["correct"] for s in summary["subjects"].values())
    assert json.loads(out.read_text()) == summary
    one = tool.run(tool.parse_args(["--param_path", str(param_dir), "--data_dir", str(data), "--subjects", "toy_words",
                                    "--split", "test", "--device", "cpu", "--dtype", "float32", "--n_shot", "0"]))
    assert one["total"] == 3 and list(one["subjects"]) == ["toy_words"]


def test_mmlu_choice_scores_are_the_log_likelihoods_of_the_letters(param_dir, tokenizer):
    from khaosz_b200 import AutoModel
    from khaosz_b200.cli.evaluate_mmlu import choice_logprobs

    model = AutoModel.from_pretrained(str(param_dir)).eval()
    context = tokenizer.encode("hello world this is a test")
    scores = choice_logprobs(model, tokenizer, context, "cpu")
    assert set(scores) == {"A", "B", "C", "D"}
    for letter in "AD":
        cont = tokenizer.encode(f" {letter}", add_special_tokens=False)
        ids = torch.tensor([context + cont])
        with torch.no_grad():
            lp = torch.log_softmax(model(ids[:, :-1])["logits"][0].float(), dim=-1)
        want = sum(float(lp[len(context) - 1 + j, tok]) for j, tok in enumerate(cont))
        assert scores[letter] == pytest.approx(want, abs=1e-4)


def test_perplexity_of_a_padded_batch_equals_the_per_text_value(param_dir, tokenizer):
    import math

    from khaosz_b200 import AutoModel
    from khaosz_b200.cli.perplexity import batch_perplexity

    model = AutoModel.from_pretrained(str(param_dir)).eval()
    texts = ["hello world this is a small test corpus", "the lazy dog", "hello"]
    got = batch_perplexity(model, tokenizer, texts, "cpu")
    for text, ppl in zip(texts, got):
        ids = torch.tensor([tokenizer.encode(text)])
        if ids.shape[1] < 2:
            assert ppl == 1.0                           # nothing to predict
            continue
        with torch.no_grad():
            lp = torch.log_softmax(model(ids[:, :-1])["logits"][0].float(), dim=-1)
        nll = -lp.gather(-1, ids[0, 1:, None]).mean()
        assert ppl == pytest.approx(math.exp(float(nll)), rel=1e-4)
