"""Batch generation over a JSONL file through ``InferenceEngine``
(reference: ``scripts/tools/generate.py:11-132``)."""

from __future__ import annotations

import argparse
import json

import torch


def parse_args(argv=None):
    p = argparse.ArgumentParser(description="Generate responses for the questions of a JSONL file")
    p.add_argument("--param_path", type=str, required=True)
    p.add_argument("--input_json_file", type=str, required=True)
    p.add_argument("--output_json_file", type=str, required=True)
    p.add_argument("--question_key", type=str, default="question")
    p.add_argument("--response_key", type=str, default="response")
    p.add_argument("--temperature", type=float, default=0.6)
    p.add_argument("--top_k", type=int, default=30)
    p.add_argument("--top_p", type=float, default=0.95)
    p.add_argument("--batch_size", type=int, default=1)
    p.add_argument("--max_tokens", type=int, default=2048)
    p.add_argument("--adapter_path", type=str, default=None, help="LoRA adapter directory, merged into the weights at load")
    p.add_argument("--device", type=str, default="cuda" if torch.cuda.is_available() else "cpu")
    return p.parse_args(argv)


def run(a) -> int:
    from ..inference import InferenceEngine
    from ..models import AutoModel
    from ..tokenize import AutoTokenizer

    tokenizer = AutoTokenizer.from_pretrained(a.param_path)
    dtype = torch.bfloat16 if a.device.startswith("cuda") else torch.float32
    model = AutoModel.from_pretrained(a.param_path).to(device=a.device, dtype=dtype).eval()
    if a.adapter_path:
        from ..models.components.lora import load_lora, merge_lora

        load_lora(model, a.adapter_path)
        merge_lora(model, unwrap=True)
    if a.device.startswith("cuda"):
        model.pack_parameters(with_grad=False)
    with open(a.input_json_file, "r", encoding="utf-8") as fh:
        items = [json.loads(line) for line in fh if line.strip()]
    done = 0
    with InferenceEngine(model, tokenizer, max_batch_size=a.batch_size, page_size=16) as engine, \
            open(a.output_json_file, "w", encoding="utf-8") as out:
        for start in range(0, len(items), a.batch_size):
            chunk = items[start:start + a.batch_size]
            prompts = [tokenizer.apply_chat_template([{"role": "user", "content": it[a.question_key]}], tokenize=False)
                       for it in chunk]
            answers = engine.generate(prompts, max_tokens=a.max_tokens, temperature=a.temperature, top_p=a.top_p,
                                      top_k=a.top_k)
            for it, ans in zip(chunk, answers):
                out.write(json.dumps({a.question_key: it[a.question_key], a.response_key: ans}, ensure_ascii=False) + "\n")
                done += 1
    return done


if __name__ == "__main__":
    print(f"generated {run(parse_args())} responses")
