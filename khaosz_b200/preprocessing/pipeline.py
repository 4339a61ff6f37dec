"""JSONL -> tokenised shards (reference: ``astrai/preprocessing/pipeline.py:38-141``).

Records are bucketed per domain; when ``max_tokens_per_shard`` tokens have accumulated every
bucket is flushed to ``<out>/<domain>/shard_NNNN`` (bin) or ``<out>/<domain>/data_NNNN.h5``.
Default dtype is int32, overridable per key through ``output.dtype``.
"""

from __future__ import annotations

import json
import logging
import os
from typing import Dict, Iterator, List, Optional

import torch
from tqdm import tqdm

from ..config.pipeline_config import PipelineConfig
from ..data.storage import save_bin, save_h5
from ..tokenize import AutoTokenizer
from .builder import DEFAULT_DOMAIN, SectionedMaskBuilder

log = logging.getLogger(__name__)

DTYPES = {name: getattr(torch, name) for name in
          ("bool", "uint8", "int8", "int16", "int32", "int64", "float16", "float32", "float64")}


def filter_by_length(text: str, min_len: int = 50, max_len: int = 2_000_000) -> bool:
    return min_len <= len(text) <= max_len


class _DomainBucket:
    """Per-domain lists of per-document values; keys that appear late are back-filled with 1s."""

    def __init__(self) -> None:
        self.columns: Dict[str, List[list]] = {}
        self.lengths: List[int] = []

    def add(self, record: Dict[str, list]) -> None:
        n = len(record["sequence"])
        for key in record:
            if key not in self.columns:
                self.columns[key] = [[1] * m for m in self.lengths]
        for key, docs in self.columns.items():
            docs.append(record.get(key) or [1] * n)
        self.lengths.append(n)

    def tensors(self, dtype_of) -> Dict[str, List[torch.Tensor]]:
        return {key: [torch.tensor([v for doc in docs for v in doc], dtype=dtype_of(key))]
                for key, docs in self.columns.items()}


class Pipeline:
    def __init__(self, config: PipelineConfig, input_paths: List[str], output_dir: str, tokenizer_path: str):
        os.makedirs(output_dir, exist_ok=True)
        self.config, self.paths = config, list(input_paths)
        self.output_dir, self.tokenizer_path = output_dir, tokenizer_path
        self.mask_builder = SectionedMaskBuilder()
        self._tokenizer = None
        self.skipped_lines = 0      # input lines that were not valid JSON

    def transform(self, item: dict) -> Optional[dict]:
        return self.mask_builder.build(item, self.config, self._tokenizer)

    def _iter_items(self) -> Iterator[dict]:
        for path in self.paths:
            with open(path, "r", encoding="utf-8") as fh:
                for number, line in enumerate(fh, 1):
                    if not line.strip():
                        continue
                    try:
                        item = json.loads(line)
                    except ValueError:       # one damaged record must not cost the whole corpus
                        item = None
                    if isinstance(item, dict):
                        yield item
                    else:
                        self.skipped_lines += 1
                        log.warning("%s:%d is not a JSON object; skipped", path, number)

    def _dtype(self, key: str) -> torch.dtype:
        return DTYPES.get((self.config.output.dtype or {}).get(key, "int32"), torch.int32)

    def _flush(self, buckets: Dict[str, _DomainBucket], shard_idx: Dict[str, int]) -> None:
        for domain, bucket in buckets.items():
            idx = shard_idx.get(domain, 0)
            tensors = bucket.tensors(self._dtype)
            root = os.path.join(self.output_dir, domain)
            if self.config.output.storage_format == "bin":
                save_bin(os.path.join(root, f"shard_{idx:04d}"), tensors)
            else:
                save_h5(root, f"data_{idx:04d}", tensors)
            shard_idx[domain] = idx + 1
            tqdm.write(f"  saved {domain}/shard_{idx:04d}  ({tensors['sequence'][0].numel():,} tokens)")

    def run(self) -> int:
        self._tokenizer = AutoTokenizer.from_pretrained(self.tokenizer_path)
        buckets: Dict[str, _DomainBucket] = {}
        shard_idx: Dict[str, int] = {}
        pending_tokens = docs = 0
        max_items = self.config.preprocessing.max_items
        for item in tqdm(self._iter_items(), desc="Tokenizing", unit="docs", mininterval=0.5):
            if max_items and docs >= max_items:
                break
            record = self.transform(item)
            if not record or not record.get("sequence"):
                continue
            domain = record.pop("domain", DEFAULT_DOMAIN)
            buckets.setdefault(domain, _DomainBucket()).add(record)
            docs += 1
            pending_tokens += len(record["sequence"])
            if pending_tokens >= self.config.output.max_tokens_per_shard:
                self._flush(buckets, shard_idx)
                buckets, pending_tokens = {}, 0
        if pending_tokens:
            self._flush(buckets, shard_idx)
        print(f"Done. {docs} documents tokenized.")
        return docs
