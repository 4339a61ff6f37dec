"""``astrai`` import names for code written against the reference framework.

``import astrai`` gives the ``khaosz_b200`` package itself, and every ``astrai.<path>`` import is
answered with the ``khaosz_b200`` module that holds the same public names (the module *objects* are
shared: ``astrai.model.AutoModel is khaosz_b200.models.AutoModel``).  Most sub-modules have the same
path in both trees; the table below lists the ones that were renamed.  Nothing is re-exported by
hand: the table is the whole compatibility layer.

Reference layout: ``astrai/__init__.py:4-34`` and the package directories of ``astrai/``.
"""

from __future__ import annotations

import importlib
import importlib.abc
import importlib.util
import sys

import khaosz_b200

# reference module path (below ``astrai.``) -> module path below ``khaosz_b200.``; longest prefix wins
RENAMED = {
    "model": "models",
    "model.components.decoder_block": "models.components.block",
    "model.components.mlp": "models.components.ffn",
    "model.components.linear": "models.components.layers",
    "model.components.embedding": "models.components.layers",
    "model.components.norm": "models.components.layers",
    "model.components.rope": "models.components.layers",
    "dataset": "data",
    "trainer.train_callback": "trainer.callbacks",
    "trainer.train_context": "trainer.context",
    "trainer.metric_util": "trainer.metrics",
    "config.preprocess_config": "config.pipeline_config",
    "parallel.module": "parallel.tensor_parallel",
}


def resolve(name: str) -> str:
    """``astrai.a.b`` -> the ``khaosz_b200`` module path that answers it."""
    assert name == "astrai" or name.startswith("astrai.")
    tail = name[len("astrai."):] if name != "astrai" else ""
    if not tail:
        return "khaosz_b200"
    parts = tail.split(".")
    for cut in range(len(parts), 0, -1):
        head = ".".join(parts[:cut])
        if head in RENAMED:
            return ".".join(["khaosz_b200", RENAMED[head], *parts[cut:]])
    return "khaosz_b200." + tail


class _AliasFinder(importlib.abc.MetaPathFinder, importlib.abc.Loader):
    def find_spec(self, fullname, path=None, target=None):
        if not fullname.startswith("astrai."):
            return None
        try:
            if importlib.util.find_spec(resolve(fullname)) is None:
                return None
        except (ImportError, AttributeError, ValueError):
            return None
        return importlib.util.spec_from_loader(fullname, self)

    def create_module(self, spec):
        return importlib.import_module(resolve(spec.name))   # the real module, under a second name

    def exec_module(self, module):
        return None


if not any(isinstance(f, _AliasFinder) for f in sys.meta_path):
    sys.meta_path.insert(0, _AliasFinder())
sys.modules[__name__] = khaosz_b200
