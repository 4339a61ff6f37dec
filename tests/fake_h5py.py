"""A small stand-in for the part of ``h5py`` that the HDF5 store uses, for hosts without the
real package: ``File(path, mode)`` as a context manager, ``create_group``, ``create_dataset(name,
data=...)``, ``keys()``, ``group[name][()]``.  A "file" is a pickled ``{group: {dataset: ndarray}}``
dictionary, so what is written by one ``File`` is read back by another from disk, as the stores and
the preprocessing pipeline expect.  Install it with ``install()`` (it refuses when the real ``h5py``
is importable, so the real one is always preferred)."""

from __future__ import annotations

import pickle
import sys
import types
from pathlib import Path

import numpy as np


class _Dataset:
    def __init__(self, array):
        self._array = np.asarray(array)

    def __getitem__(self, key):
        return self._array if key == () else self._array[key]

    @property
    def shape(self):
        return self._array.shape

    @property
    def dtype(self):
        return self._array.dtype


class _Group:
    def __init__(self, items=None):
        self._items = {} if items is None else items

    def create_dataset(self, name, data=None, **_):
        self._items[name] = np.array(data)
        return _Dataset(self._items[name])

    def keys(self):
        return self._items.keys()

    def __iter__(self):
        return iter(self._items)

    def __len__(self):
        return len(self._items)

    def __contains__(self, name):
        return name in self._items

    def __getitem__(self, name):
        return _Dataset(self._items[name])


class File:
    def __init__(self, path, mode="r"):
        self._path, self._mode = Path(path), mode
        self._groups = {}
        if mode.startswith("r") or mode == "a":
            if self._path.exists():
                with open(self._path, "rb") as fh:
                    self._groups = pickle.load(fh)
            elif mode.startswith("r"):
                raise FileNotFoundError(str(self._path))

    def create_group(self, name):
        self._groups[name] = {}
        return _Group(self._groups[name])

    def keys(self):
        return self._groups.keys()

    def __iter__(self):
        return iter(self._groups)

    def __contains__(self, name):
        return name in self._groups

    def __getitem__(self, name):
        return _Group(self._groups[name])

    def close(self):
        if self._mode != "r":
            with open(self._path, "wb") as fh:
                pickle.dump(self._groups, fh)

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()
        return False


def install() -> bool:
    """Register this module as ``h5py`` unless the real package exists.  Returns True when installed."""
    try:
        import h5py  # noqa: F401

        return getattr(sys.modules["h5py"], "__fake__", False)
    except ImportError:
        mod = types.ModuleType("h5py")
        mod.File = File
        mod.__fake__ = True
        sys.modules["h5py"] = mod
        return True
