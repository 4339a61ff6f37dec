"""Perplexity of the texts of a JSONL file (reference: ``scripts/tools/perplexity.py:12-111``).
Padded batches; the per-token log-probabilities come from the fused kernel on CUDA."""

from __future__ import annotations

import argparse
import json
import math

import torch

from .. import ops


def parse_args(argv=None):
    p = argparse.ArgumentParser(description="Per-text perplexity")
    p.add_argument("--param_path", type=str, required=True)
    p.add_argument("--input_file", type=str, required=True)
    p.add_argument("--output_file", type=str, required=True)
    p.add_argument("--batch_size", type=int, default=4)
    p.add_argument("--text_key", type=str, default="text")
    p.add_argument("--adapter_path", type=str, default=None, help="LoRA adapter directory, merged into the weights at load")
    p.add_argument("--device", type=str, default="cuda" if torch.cuda.is_available() else "cpu")
    return p.parse_args(argv)


@torch.inference_mode()
def batch_perplexity(model, tokenizer, texts, device, max_len=None):
    encoded = [tokenizer.encode(t)[: max_len or model.config.max_len] for t in texts]
    width = max(len(e) for e in encoded)
    pad = tokenizer.pad_token_id if tokenizer.pad_token_id is not None else 0
    ids = torch.full((len(encoded), width), pad, dtype=torch.long, device=device)
    mask = torch.zeros((len(encoded), width), dtype=torch.bool, device=device)
    for i, e in enumerate(encoded):
        ids[i, :len(e)] = torch.tensor(e, device=device)
        mask[i, :len(e)] = True
    logits = model(ids[:, :-1].contiguous(), mask[:, :-1])["logits"]
    lp = ops.token_logprobs(logits, ids[:, 1:].contiguous()) * mask[:, 1:]
    nll = -lp.sum(dim=-1) / mask[:, 1:].sum(dim=-1).clamp(min=1)
    return [math.exp(min(v, 50.0)) for v in nll.tolist()]


def run(a):
    from ..models import AutoModel
    from ..tokenize import AutoTokenizer

    tokenizer = AutoTokenizer.from_pretrained(a.param_path)
    dtype = torch.bfloat16 if a.device.startswith("cuda") else torch.float32
    model = AutoModel.from_pretrained(a.param_path).to(device=a.device, dtype=dtype).eval()
    if a.adapter_path:
        from ..models.components.lora import load_lora, merge_lora

        load_lora(model, a.adapter_path)
        merge_lora(model, unwrap=True)
    with open(a.input_file, "r", encoding="utf-8") as fh:
        items = [json.loads(line) for line in fh if line.strip()]
    with open(a.output_file, "w", encoding="utf-8") as out:
        for s in range(0, len(items), a.batch_size):
            chunk = items[s:s + a.batch_size]
            for it, ppl in zip(chunk, batch_perplexity(model, tokenizer, [it[a.text_key] for it in chunk], a.device)):
                out.write(json.dumps({a.text_key: it[a.text_key], "ppl": ppl}, ensure_ascii=False) + "\n")
    return len(items)


if __name__ == "__main__":
    print(f"scored {run(parse_args())} texts")
