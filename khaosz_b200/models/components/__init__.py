from .attention import GQA, MLA, AttnFactory
from .block import DecoderBlock
from .ffn import MLP, DeepSeekMoE, FFNFactory
from .layers import Embedding, Linear, RMSNorm, RotaryEmbedding
from .lora import LoRAConfig, LoRALinear, inject_lora, load_lora, merge_lora, save_lora

__all__ = ["GQA", "MLA", "AttnFactory", "DecoderBlock", "MLP", "DeepSeekMoE", "FFNFactory", "Embedding", "Linear",
           "RMSNorm", "RotaryEmbedding", "LoRAConfig", "LoRALinear", "inject_lora", "load_lora", "merge_lora",
           "save_lora"]
