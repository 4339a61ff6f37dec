"""Preprocessing CLI: JSONL files -> token shards (reference: ``scripts/tools/preprocess.py:9-34``)."""

from __future__ import annotations

import argparse

from ..config import PipelineConfig
from ..preprocessing import Pipeline


def parse_args(argv=None):
    p = argparse.ArgumentParser(description="Tokenise JSONL files into training shards")
    p.add_argument("inputs", nargs="+", help="Input JSONL files")
    p.add_argument("--output_dir", "-o", required=True)
    p.add_argument("--config", "-c", required=True, help="Pipeline config JSON")
    p.add_argument("--tokenizer_path", default="params")
    return p.parse_args(argv)


def main(argv=None):
    a = parse_args(argv)
    return Pipeline(PipelineConfig.from_json(a.config), a.inputs, a.output_dir, a.tokenizer_path).run()


if __name__ == "__main__":
    main()
