"""MMLU by log-likelihood ranking of the four answer letters
(reference: ``scripts/tools/evaluate_mmlu.py:80-291``).  ``--download`` needs network access;
offline, point ``--data_dir`` at an extracted copy (``dev/`` and ``test/`` or ``val/`` CSVs)."""

from __future__ import annotations

import argparse
import csv
import json
import os
from typing import Dict, List, Optional

import torch

from .. import ops

MMLU_URL = "https://people.eecs.berkeley.edu/~hendrycks/data.tar"
LETTERS = ("A", "B", "C", "D")


def download_mmlu(data_dir: str) -> None:
    import shutil
    import tarfile

    import requests

    os.makedirs(data_dir, exist_ok=True)
    tar_path = os.path.join(data_dir, "data.tar")
    with requests.get(MMLU_URL, stream=True, timeout=300) as resp:
        resp.raise_for_status()
        with open(tar_path, "wb") as fh:
            for chunk in resp.iter_content(chunk_size=1 << 16):
                fh.write(chunk)
    with tarfile.open(tar_path, "r") as tf:
        tf.extractall(data_dir)
    os.remove(tar_path)
    inner = os.path.join(data_dir, "data")
    if os.path.isdir(inner):
        for name in os.listdir(inner):
            dst = os.path.join(data_dir, name)
            if os.path.isdir(dst):
                shutil.rmtree(dst)
            elif os.path.exists(dst):
                os.remove(dst)
            os.rename(os.path.join(inner, name), dst)
        os.rmdir(inner)


def load_csv(path: str) -> List[dict]:
    rows = []
    with open(path, "r", encoding="utf-8") as fh:
        for row in csv.reader(fh):
            if len(row) < 6 or row[0].strip().lower() == "question":
                continue
            item = {"question": row[0].strip(), "answer": row[5].strip()}
            for letter, cell in zip(LETTERS, row[1:5]):
                cell = cell.strip()
                item[letter] = cell[2:].strip() if cell.startswith(f"{letter})") else cell
            rows.append(item)
    return rows


def format_question(item: dict, with_answer: bool) -> str:
    lines = [f"Question: {item['question']}"] + [f"{k}. {item[k]}" for k in LETTERS]
    lines.append(f"Answer: {item['answer']}\n" if with_answer else "Answer:")
    return "\n".join(lines)


def build_prompt(question: str, choices: dict, subject: str, n_shot: int, dev_data: List[dict]) -> str:
    parts = []
    if n_shot > 0 and dev_data:
        parts.append(f"The following are multiple choice questions (with answers) about {subject}.\n")
        parts += [format_question(ex, True) for ex in dev_data[:n_shot]]
    parts.append(format_question({"question": question, **{k: choices[k] for k in LETTERS}}, False))
    return "\n".join(parts)


@torch.inference_mode()
def choice_logprobs(model, tokenizer, context_ids: List[int], device) -> Dict[str, float]:
    """Log-likelihood of `` A`` .. `` D`` after the context; the four continuations run as one batch."""
    conts = {k: tokenizer.encode(f" {k}", add_special_tokens=False) for k in LETTERS}
    max_len = model.config.max_len
    rows, spans = [], []
    width = 0
    for k in LETTERS:
        ids = (context_ids + conts[k])[-max_len:]
        rows.append(ids)
        spans.append((len(ids) - len(conts[k]), len(ids)))
        width = max(width, len(ids))
    batch = torch.zeros((4, width), dtype=torch.long, device=device)
    for i, ids in enumerate(rows):
        batch[i, :len(ids)] = torch.tensor(ids, device=device)
    logits = model(batch[:, :-1].contiguous())["logits"]
    lp = ops.token_logprobs(logits, batch[:, 1:].contiguous())
    return {k: float(lp[i, spans[i][0] - 1:spans[i][1] - 1].sum()) for i, k in enumerate(LETTERS)}


def evaluate_subject(model, tokenizer, subject: str, test_data: List[dict], dev_data: Optional[List[dict]], device,
                     n_shot: int):
    correct = 0
    for item in test_data:
        prompt = build_prompt(item["question"], item, subject.replace("_", " "), n_shot, dev_data or [])
        scores = choice_logprobs(model, tokenizer, tokenizer.encode(prompt), device)
        correct += int(max(scores, key=scores.get) == item["answer"])
    total = len(test_data)
    return (correct / total if total else 0.0), correct, total


def parse_args(argv=None):
    p = argparse.ArgumentParser(description="MMLU evaluation")
    p.add_argument("--param_path", type=str, default="./params")
    p.add_argument("--data_dir", type=str, default="./mmlu_data")
    p.add_argument("--download", action="store_true")
    p.add_argument("--n_shot", type=int, default=5)
    p.add_argument("--subjects", type=str, nargs="+")
    p.add_argument("--output", type=str)
    p.add_argument("--split", type=str, default="test", choices=["test", "val"])
    p.add_argument("--device", type=str, default="cuda" if torch.cuda.is_available() else "cpu")
    p.add_argument("--dtype", type=str, default="bfloat16", choices=["bfloat16", "float16", "float32"])
    return p.parse_args(argv)


def run(a) -> dict:
    from ..models import AutoModel
    from ..tokenize import AutoTokenizer

    if a.download:
        download_mmlu(a.data_dir)
    tokenizer = AutoTokenizer.from_pretrained(a.param_path)
    model = AutoModel.from_pretrained(a.param_path).to(device=a.device, dtype=getattr(torch, a.dtype)).eval()
    split_dir = os.path.join(a.data_dir, a.split)
    subjects = a.subjects or sorted(f[: -len(f"_{a.split}.csv")] for f in os.listdir(split_dir) if f.endswith(".csv"))
    results, hit, seen = {}, 0, 0
    for subject in subjects:
        test = load_csv(os.path.join(split_dir, f"{subject}_{a.split}.csv"))
        dev_path = os.path.join(a.data_dir, "dev", f"{subject}_dev.csv")
        dev = load_csv(dev_path) if os.path.exists(dev_path) else None
        acc, c, t = evaluate_subject(model, tokenizer, subject, test, dev, a.device, a.n_shot)
        results[subject] = {"accuracy": acc, "correct": c, "total": t}
        hit, seen = hit + c, seen + t
        print(f"{subject:45s} {acc:.4f} ({c}/{t})")
    summary = {"average": hit / seen if seen else 0.0, "correct": hit, "total": seen, "subjects": results}
    print(f"average accuracy: {summary['average']:.4f}")
    if a.output:
        with open(a.output, "w", encoding="utf-8") as fh:
            json.dump(summary, fh, indent=2)
    return summary


if __name__ == "__main__":
    run(parse_args())
