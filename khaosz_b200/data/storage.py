"""Token storage: HDF5 and flat-binary (memory-mapped) shards behind one ``Store`` interface.

File formats are the reference's (``astrai/dataset/storage.py:36-131``):

* bin: ``<dir>/<key>.bin`` (all segments of a key concatenated) + ``<dir>/meta.json``
  ``{key: {"shape": [...], "dtype": "int32"}}``; read with ``np.memmap``
* h5:  one group per key holding datasets ``data_0 .. data_n``

``h5py`` is imported lazily, so everything else works on hosts without it.
"""

from __future__ import annotations

import bisect
import json
from abc import ABC, abstractmethod
from pathlib import Path
from typing import Dict, List, Sequence, Union

import numpy as np
import torch
from torch import Tensor

from ..factory import BaseFactory

H5_SUFFIXES = (".h5", ".hdf5")
BIN_SUFFIX = ".bin"
META_NAME = "meta.json"


def _h5py():
    try:
        import h5py
    except ImportError as exc:  # pragma: no cover - depends on the host
        raise ImportError("the h5 storage format needs the 'h5py' package") from exc
    return h5py


# -- writers / readers --------------------------------------------------------------------
def save_h5(file_path: str, file_name: str, tensor_group: Dict[str, List[Tensor]]) -> None:
    h5py = _h5py()
    root = Path(file_path)
    root.mkdir(parents=True, exist_ok=True)
    with h5py.File(root / f"{file_name}.h5", "w") as fh:
        for key, tensors in tensor_group.items():
            grp = fh.create_group(key)
            for i, t in enumerate(tensors):
                grp.create_dataset(f"data_{i}", data=t.cpu().numpy())


def load_h5(file_path: str, share_memory: bool = True) -> Dict[str, List[Tensor]]:
    h5py = _h5py()
    out: Dict[str, List[Tensor]] = {}
    root = Path(file_path)
    files = [root] if root.is_file() else sorted(p for s in H5_SUFFIXES for p in root.rglob(f"*{s}"))
    for path in files:
        with h5py.File(path, "r") as fh:
            for key in fh.keys():
                for name in sorted(fh[key].keys(), key=lambda n: int(n.rsplit("_", 1)[-1])):
                    t = torch.from_numpy(fh[key][name][()])
                    out.setdefault(key, []).append(t.share_memory_() if share_memory else t)
    return out


def save_bin(file_path: str, tensor_group: Dict[str, List[Tensor]]) -> None:
    root = Path(file_path)
    root.mkdir(parents=True, exist_ok=True)
    meta = {}
    for key, tensors in tensor_group.items():
        flat = torch.cat([t.reshape(-1) for t in tensors]).cpu().numpy()
        flat.tofile(root / f"{key}{BIN_SUFFIX}")
        meta[key] = {"shape": list(flat.shape), "dtype": str(flat.dtype)}
    (root / META_NAME).write_text(json.dumps(meta))


def load_bin(file_path: str) -> Dict[str, List[Tensor]]:
    root = Path(file_path)
    meta = json.loads((root / META_NAME).read_text())
    out: Dict[str, List[Tensor]] = {}
    for key, info in meta.items():
        arr = np.memmap(root / f"{key}{BIN_SUFFIX}", dtype=np.dtype(info["dtype"]), mode="r+",
                        shape=tuple(info["shape"]))
        out[key] = [torch.from_numpy(arr)]
    return out


def detect_format(load_path: str) -> str:
    """``"h5"`` or ``"bin"`` from a file suffix or a recursive directory scan (h5 wins)."""
    root = Path(load_path)
    if root.is_file():
        if root.suffix in H5_SUFFIXES:
            return "h5"
        if root.suffix == BIN_SUFFIX:
            return "bin"
        raise ValueError(f"Unsupported storage file: {root}")
    if root.is_dir():
        if any(True for s in H5_SUFFIXES for _ in root.rglob(f"*{s}")):
            return "h5"
        if any(True for _ in root.rglob(f"*{BIN_SUFFIX}")) or any(True for _ in root.rglob(META_NAME)):
            return "bin"
    raise FileNotFoundError(f"No supported data files found under {load_path}")


# -- stores ---------------------------------------------------------------------------------
class Store(ABC):
    """key -> list of 1-D segments, addressed as one virtual sequence per key."""

    def __init__(self) -> None:
        self._segments: Dict[str, List[Tensor]] = {}
        self._ends: Dict[str, List[int]] = {}
        self._length = 0
        self._loaded = False

    @abstractmethod
    def load(self, load_path: str) -> None: ...

    def _install(self, segments: Dict[str, List[Tensor]]) -> None:
        self._segments, self._ends = {}, {}
        lengths = []
        for key, tensors in segments.items():
            ends, total = [], 0
            for t in tensors:
                total += int(t.shape[0])
                ends.append(total)
            self._segments[key], self._ends[key] = list(tensors), ends
            lengths.append(total)
        self._length = min(lengths) if lengths else 0
        self._loaded = True

    _normalize = _install   # the reference's name for the same step (``astrai/dataset/storage.py:193``)

    @property
    def keys(self) -> List[str]:
        return list(self._segments)

    def __len__(self) -> int:
        return self._length

    def _slice(self, key: str, begin: int, end: int) -> Tensor:
        segs, ends = self._segments[key], self._ends[key]
        if begin == end:
            return segs[0][:0] if segs else torch.empty(0, dtype=torch.long)
        first = bisect.bisect_right(ends, begin)
        last = bisect.bisect_left(ends, end)
        parts = []
        for i in range(first, last + 1):
            base = ends[i - 1] if i else 0
            parts.append(segs[i][max(begin - base, 0):min(end - base, segs[i].shape[0])])
        return parts[0] if len(parts) == 1 else torch.cat(parts)

    def fetch(self, begin_idx: int, end_idx: int, keys: Union[str, Sequence[str]]):
        if not self._loaded:
            raise RuntimeError("Store not loaded, call load() first")
        if not (0 <= begin_idx < self._length and 0 <= end_idx <= self._length):
            raise ValueError(f"Index out of bounds: [{begin_idx}, {end_idx}) for length {self._length}")
        if isinstance(keys, str):
            return self._slice(keys, begin_idx, end_idx)
        return {k: self._slice(k, begin_idx, end_idx) for k in keys}


class StoreFactory(BaseFactory[Store]):
    pass


@StoreFactory.register("h5")
class H5Store(Store):
    def load(self, load_path: str) -> None:
        self._install(load_h5(load_path))


@StoreFactory.register("bin")
class MmapStore(Store):
    """Merges every ``meta.json`` directory found under the path (shards in sorted order)."""

    def load(self, load_path: str) -> None:
        root = Path(load_path)
        if root.is_file():
            root = root.parent
        dirs = sorted(p.parent for p in root.rglob(META_NAME))
        if not dirs:
            raise FileNotFoundError(f"No {META_NAME} found under {load_path}")
        merged: Dict[str, List[Tensor]] = {}
        for d in dirs:
            for key, tensors in load_bin(str(d)).items():
                merged.setdefault(key, []).extend(tensors)
        self._install(merged)
