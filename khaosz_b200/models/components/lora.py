"""Low-rank adapters for the bias-free ``Linear`` layers.

Same user-visible behaviour as ``astrai/model/components/lora.py:31-194``: the wrapped layer
shares (and freezes) the base weight, ``lora_A: [r, in] ~ N(0,1)/r``, ``lora_B: [out, r] = 0``,
scaling ``alpha / r``; adapters are saved as ``adapter_model.safetensors`` +
``adapter_config.json {r, alpha, target_modules}``.
"""

from __future__ import annotations

import logging
from dataclasses import asdict, dataclass
from pathlib import Path
from typing import Dict, Iterable, List, Optional, Set

import torch
import torch.nn as nn

from ... import ops
from ...serialization import load_json, load_state_dict, save_json, save_safetensors
from .layers import Linear

log = logging.getLogger(__name__)

TARGET_MODULES_ATTN = frozenset({"q_proj", "k_proj", "v_proj", "o_proj"})
TARGET_MODULES_FFN = frozenset({"up", "gate", "down"})
ADAPTER_WEIGHTS = "adapter_model.safetensors"
ADAPTER_CONFIG = "adapter_config.json"


@dataclass
class LoRAConfig:
    r: int = 16
    alpha: int = 32
    target_modules: tuple = ("q_proj", "v_proj")


class LoRALinear(nn.Module):
    def __init__(self, base: Linear, r: int = 16, alpha: int = 32):
        super().__init__()
        self.weight = base.weight  # shared storage with the wrapped layer
        self.weight.requires_grad_(False)
        self.bias = base.bias
        if self.bias is not None:
            self.bias.requires_grad_(False)
        out_dim, in_dim = self.weight.shape
        self.r, self.scaling = r, alpha / r
        kw = dict(device=self.weight.device, dtype=self.weight.dtype)
        self.lora_A = nn.Parameter(torch.randn(r, in_dim, **kw) / r)
        self.lora_B = nn.Parameter(torch.zeros(out_dim, r, **kw))
        self._merged = False

    def forward(self, x: torch.Tensor, residual: Optional[torch.Tensor] = None) -> torch.Tensor:
        y = ops.linear(x, self.weight, residual)
        if self.bias is not None:
            y = y + self.bias
        if self._merged:
            return y
        return y + (x @ self.lora_A.t()) @ self.lora_B.t() * self.scaling

    def merge(self) -> None:
        if self._merged:
            return
        with torch.no_grad():
            self.weight.add_((self.lora_B @ self.lora_A) * self.scaling)
        self._merged = True
        del self.lora_A
        del self.lora_B


def _linear_children(model: nn.Module) -> Dict[str, List[str]]:
    found: Dict[str, List[str]] = {}
    for path, mod in model.named_modules():
        if isinstance(mod, Linear):
            found.setdefault(path.rpartition(".")[2], []).append(path)
    return found


_collect_lora_info = _linear_children   # the reference's name (``astrai/model/components/lora.py:61``)


def _adapters(model: nn.Module) -> List[LoRALinear]:
    return [m for m in model.modules() if isinstance(m, LoRALinear)]


def _get_lora_count(model: nn.Module) -> int:
    return len(_adapters(model))


def inject_lora(model: nn.Module, r: int = 16, alpha: int = 32, target_modules: Optional[Iterable[str]] = None) -> LoRAConfig:
    """Wrap every ``Linear`` whose attribute name is in ``target_modules`` (default: the four
    attention projections).  Already wrapped layers are left alone."""
    targets: Set[str] = set(TARGET_MODULES_ATTN if target_modules is None else target_modules)
    candidates = _linear_children(model)
    count = 0
    for leaf in sorted(targets & set(candidates)):
        for path in candidates[leaf]:
            parent_path = path.rpartition(".")[0]
            parent = model.get_submodule(parent_path) if parent_path else model
            setattr(parent, leaf, LoRALinear(getattr(parent, leaf), r=r, alpha=alpha))
            count += 1
    if count:
        log.info("LoRA injected: %d layers (r=%d, alpha=%d)", count, r, alpha)
    else:
        log.warning("No LoRA layers injected. Available Linear child names: %s. target_modules: %s.",
                    sorted(candidates), sorted(targets))
    return LoRAConfig(r=r, alpha=alpha, target_modules=tuple(targets))


def merge_lora(model: nn.Module, unwrap: bool = False) -> None:
    """Fold every adapter into its base weight.  ``unwrap=True`` also puts plain ``Linear`` layers
    (sharing the merged weights) back in place of the wrappers, so the model is again the
    architecture the packed-projection and tensor-parallel paths expect."""
    layers = _adapters(model)
    for layer in layers:
        layer.merge()
    if layers:
        log.info("Merged %d LoRA layers", len(layers))
    else:
        log.warning("No LoRA layers to merge.")
    if unwrap:
        for path, mod in list(model.named_modules()):
            if isinstance(mod, LoRALinear):
                plain = Linear.__new__(Linear)
                nn.Module.__init__(plain)
                plain.out_dim, plain.in_dim = mod.weight.shape
                plain.weight, plain.bias = mod.weight, mod.bias
                parent_path, _, leaf = path.rpartition(".")
                setattr(model.get_submodule(parent_path) if parent_path else model, leaf, plain)


def save_lora(model: nn.Module, save_dir: str, config: LoRAConfig) -> None:
    tensors = {k: v for k, v in model.state_dict().items() if k.rpartition(".")[2] in ("lora_A", "lora_B")}
    if not tensors:
        raise RuntimeError("No LoRA parameters found in model (not injected, or already merged).")
    root = Path(save_dir)
    root.mkdir(parents=True, exist_ok=True)
    save_safetensors(tensors, root / ADAPTER_WEIGHTS)
    save_json(asdict(config), root / ADAPTER_CONFIG)


def load_lora(model: nn.Module, load_dir: str) -> LoRAConfig:
    root = Path(load_dir)
    raw = load_json(root / ADAPTER_CONFIG)
    config = LoRAConfig(r=raw["r"], alpha=raw["alpha"], target_modules=tuple(raw["target_modules"]))
    if _adapters(model):
        log.warning("Model already has LoRA layers; loading adapter weights onto them.")
    else:
        inject_lora(model, r=config.r, alpha=config.alpha, target_modules=set(config.target_modules))
    weights = load_state_dict(root / ADAPTER_WEIGHTS)
    try:
        missing, unexpected = model.load_state_dict(weights, strict=False)
    except RuntimeError as exc:
        if "size mismatch" in str(exc):
            raise RuntimeError(f"LoRA size mismatch: adapter rank r={config.r} does not fit the injected "
                               f"layers. Original error: {exc}") from exc
        raise
    if not _adapters(model):
        raise RuntimeError("No LoRA layers found after loading.")
    absent = [k for k in missing if "lora_" in k]
    if absent:
        raise RuntimeError(f"LoRA weight keys not found in adapter: {absent}")
    if unexpected:
        log.warning("LoRA load: %d unexpected keys", len(unexpected))
    return config
