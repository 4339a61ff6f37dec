"""Interactive demos: ``python -m khaosz_b200.cli.demo {complete,batch,chat,download} --param_path DIR``.

Counterparts of the reference's ``scripts/demo/{generate_ar,generate_batch,stream_chat,download}.py``
as sub-commands of one tool.  ``download`` needs ``huggingface_hub`` and network access.
"""

from __future__ import annotations

import argparse
import sys
from pathlib import Path


def _engine(param_path: str, device: str, max_batch_size: int = 1):
    import torch

    from ..inference import InferenceEngine
    from ..models import AutoModel
    from ..tokenize import AutoTokenizer

    model = AutoModel.from_pretrained(param_path)
    tokenizer = AutoTokenizer.from_pretrained(param_path)
    model.to(device=device, dtype=torch.bfloat16 if device.startswith("cuda") else torch.float32)
    return InferenceEngine(model=model, tokenizer=tokenizer, max_batch_size=max_batch_size), tokenizer


def _sampling(args) -> dict:
    return dict(max_tokens=args.max_tokens, temperature=args.temperature, top_p=args.top_p, top_k=args.top_k)


def complete(args) -> None:
    """Stream the continuation of one prompt read from stdin."""
    engine, _ = _engine(args.param_path, args.device)
    try:
        prompt = input(">> ")
        for piece in engine.generate(prompt=prompt, stream=True, **_sampling(args)):
            print(piece, end="", flush=True)
        print()
    finally:
        engine.shutdown()


def batch(args) -> None:
    """Complete several prompts (one per line on stdin, empty line ends) as one batch."""
    prompts = []
    for line in sys.stdin:
        line = line.rstrip("\n")
        if not line:
            break
        prompts.append(line)
    if not prompts:
        return
    engine, _ = _engine(args.param_path, args.device, max_batch_size=len(prompts))
    try:
        for prompt, text in zip(prompts, engine.generate(prompt=prompts, stream=False, **_sampling(args))):
            print(f"### {prompt}\n{text}\n")
    finally:
        engine.shutdown()


def chat(args) -> None:
    """Multi-turn chat through the tokenizer's chat template; ``!exit`` leaves."""
    engine, tokenizer = _engine(args.param_path, args.device)
    history = [{"role": "system", "content": args.system}]
    try:
        while True:
            query = input(">> ")
            if query.strip() == "!exit":
                break
            history.append({"role": "user", "content": query})
            prompt = tokenizer.apply_chat_template(history, tokenize=False)
            answer = []
            for piece in engine.generate(prompt=prompt, stream=True, **_sampling(args)):
                print(piece, end="", flush=True)
                answer.append(piece)
            print()
            history.append({"role": "assistant", "content": "".join(answer).strip()})
    finally:
        engine.shutdown()


def download(args) -> None:
    try:
        from huggingface_hub import snapshot_download
    except ImportError as exc:  # pragma: no cover - optional dependency
        raise SystemExit("huggingface_hub is not installed") from exc
    target = Path(args.param_path)
    if target.exists() and any(target.iterdir()) and not args.force:
        print(f"{target} is not empty; use --force to download again")
        return
    snapshot_download(repo_id=args.repo_id, local_dir=str(target))


def main(argv=None) -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("command", choices=["complete", "batch", "chat", "download"])
    ap.add_argument("--param_path", default="params")
    ap.add_argument("--device", default="cuda")
    ap.add_argument("--max_tokens", type=int, default=2048)
    ap.add_argument("--temperature", type=float, default=0.8)
    ap.add_argument("--top_p", type=float, default=0.95)
    ap.add_argument("--top_k", type=int, default=50)
    ap.add_argument("--system", default="You are a helpful assistant.")
    ap.add_argument("--repo_id", default="ViperEk/KHAOSZ")
    ap.add_argument("--force", action="store_true")
    args = ap.parse_args(argv)
    {"complete": complete, "batch": batch, "chat": chat, "download": download}[args.command](args)


if __name__ == "__main__":
    main()
