from .automodel import AutoModel
from .components import (GQA, MLA, MLP, AttnFactory, DecoderBlock, DeepSeekMoE, Embedding, FFNFactory, Linear,
                         LoRAConfig, LoRALinear, RMSNorm, RotaryEmbedding, inject_lora, load_lora, merge_lora,
                         save_lora)
from .encoder import EmbeddingEncoder
from .transformer import AutoRegressiveLM, process_attention_mask

__all__ = ["AutoModel", "AutoRegressiveLM", "EmbeddingEncoder", "process_attention_mask", "GQA", "MLA", "MLP",
           "AttnFactory", "DecoderBlock", "DeepSeekMoE", "Embedding", "FFNFactory", "Linear", "LoRAConfig",
           "LoRALinear", "RMSNorm", "RotaryEmbedding", "inject_lora", "load_lora", "merge_lora", "save_lora"]
