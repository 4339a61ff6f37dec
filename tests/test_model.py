import logging
import os

import pytest
import torch

from conftest import tiny_config
from khaosz_b200 import AutoModel, AutoRegressiveLM, EncoderConfig
from khaosz_b200.models import (EmbeddingEncoder, LoRAConfig, LoRALinear, inject_lora, load_lora, merge_lora,
                                process_attention_mask, save_lora)
from khaosz_b200.models.components.layers import Linear, RotaryEmbedding, ntk_scaled_base

VARIANTS = {
    "gqa_mlp": {},
    "mla_mlp": dict(attn_type="mla", n_heads=2, n_kv_heads=1, dim=8, dim_ffn=16, kv_lora_rank=4, qk_nope_head_dim=2,
                    qk_rope_head_dim=2),
    "gqa_moe": dict(ffn_type="moe", n_routed_experts=4, n_shared_experts=1, n_activated_experts=2),
    "rope_theta": dict(rope_theta=50000.0, rope_scaling={"type": "ntk", "factor": 2.0}),
    "qk_norm_gate": dict(use_qk_norm=True, use_gated_attention=True),
    "tie_weight": dict(tie_weight=True),
}


@pytest.mark.parametrize("name", sorted(VARIANTS))
def test_forward_variants(name):
    cfg = tiny_config(**VARIANTS[name])
    model = AutoRegressiveLM(cfg)
    ids = torch.randint(0, cfg.vocab_size, (2, 12))
    out = model(ids)
    assert out["logits"].shape == (2, 12, cfg.vocab_size) and out["hidden_states"].shape == (2, 12, cfg.dim)
    assert not out["logits"].isnan().any()
    out["logits"].sum().backward()
    assert all(p.grad is not None for p in model.parameters() if p.requires_grad)
    # padding mask + explicit positions variant
    mask = torch.ones(2, 12, dtype=torch.bool)
    mask[1, 8:] = False
    pos = torch.arange(12).unsqueeze(0).expand(2, 12)
    assert not model(ids, input_mask=mask, position_ids=pos)["logits"].isnan().any()


def test_causality():
    model = AutoRegressiveLM(tiny_config()).eval()
    ids = torch.randint(0, 300, (1, 10))
    a = model(ids)["logits"]
    ids2 = ids.clone()
    ids2[0, 7] = (ids2[0, 7] + 1) % 300
    b = model(ids2)["logits"]
    assert torch.allclose(a[0, :7], b[0, :7], atol=1e-6) and not torch.allclose(a[0, 7:], b[0, 7:])


def test_process_attention_mask_semantics():
    x = torch.zeros(2, 4, 8)
    assert process_attention_mask(x, None, torch.ones(2, 4)) is None  # ignored without positions
    pos = torch.arange(4).unsqueeze(0).expand(2, 4)
    assert process_attention_mask(x, pos, None, is_causal=True) is None
    pad = torch.tensor([[1, 1, 1, 1], [1, 1, 0, 0]], dtype=torch.bool)
    m = process_attention_mask(x, pos, pad, is_causal=True)
    assert m.shape == (2, 1, 4, 4) and m[0, 0, 0, 1] < -1e30 and m[0, 0, 1, 0] == 0 and m[1, 0, 3, 2] < -1e30
    four_d = torch.zeros(2, 1, 4, 4)
    assert process_attention_mask(x, pos, four_d) is four_d


def test_rope_ntk_and_table():
    assert ntk_scaled_base(10000.0, 2.0, 64) == pytest.approx(10000.0 * 2.0 ** (64 / 62))
    r = RotaryEmbedding(8, 16, 10000.0)
    assert r.cos_sin.shape == (16, 4, 2) and "cos_sin" not in r.state_dict()
    assert torch.allclose(r.cos_sin[0, :, 0], torch.ones(4)) and torch.allclose(r.cos_sin[0, :, 1], torch.zeros(4))


def test_tied_weights_state_dict_semantics(tmp_path):
    tied = AutoRegressiveLM(tiny_config(tie_weight=True))
    assert tied.lm_head.weight.data_ptr() == tied.embed_tokens.weight.data_ptr()
    sd = tied.state_dict()
    assert "lm_head.weight" not in sd and "embed_tokens.weight" in sd
    tied.save_pretrained(str(tmp_path / "tied"))
    again = AutoModel.from_pretrained(str(tmp_path / "tied"))
    assert isinstance(again, AutoRegressiveLM) and torch.equal(again.embed_tokens.weight, tied.embed_tokens.weight)
    assert again.lm_head.weight.data_ptr() == again.embed_tokens.weight.data_ptr()
    untied = AutoRegressiveLM(tiny_config(tie_weight=False))
    untied.load_state_dict(sd)  # tied checkpoint into an untied model: embedding copied
    assert torch.equal(untied.lm_head.weight, untied.embed_tokens.weight)
    assert untied.lm_head.weight.data_ptr() != untied.embed_tokens.weight.data_ptr()
    assert "lm_head.weight" in untied.state_dict()


def test_state_dict_key_names():
    keys = set(AutoRegressiveLM(tiny_config(use_qk_norm=True, use_gated_attention=True)).state_dict())
    for k in ("embed_tokens.weight", "layers.0.attention.q_proj.weight", "layers.0.attention.k_proj.weight",
              "layers.0.attention.v_proj.weight", "layers.0.attention.o_proj.weight", "layers.0.attention.q_norm.weight",
              "layers.0.attention.k_norm.weight", "layers.0.attention.gate.weight", "layers.0.input_norm.weight",
              "layers.0.post_attention_norm.weight", "layers.1.mlp.up.weight", "layers.1.mlp.gate.weight",
              "layers.1.mlp.down.weight", "norm.weight", "lm_head.weight"):
        assert k in keys, k
    moe = set(AutoRegressiveLM(tiny_config(ffn_type="moe", n_routed_experts=2, n_shared_experts=1,
                                           n_activated_experts=1)).state_dict())
    assert {"layers.0.mlp.router.weight", "layers.0.mlp.shared_experts.0.up.weight",
            "layers.0.mlp.routed_experts.1.down.weight"} <= moe


def test_from_pretrained_errors_and_random_init_skip(tmp_path):
    with pytest.raises(FileNotFoundError):
        AutoModel.from_pretrained(str(tmp_path))
    cfg = tiny_config()
    cfg.to_file(str(tmp_path / "config.json"))
    model = AutoModel.from_pretrained(str(tmp_path))  # config only: allowed
    assert isinstance(model, AutoRegressiveLM)
    assert torch.nn.init.normal_.__name__ == "normal_"  # init functions restored


def test_packed_parameters_keep_outputs():
    model = AutoRegressiveLM(tiny_config()).eval()
    ids = torch.randint(0, 300, (2, 9))
    before = model(ids)["logits"]
    flat = model.pack_parameters(with_grad=True)
    att = model.layers[0].attention
    assert att.k_proj.weight.data_ptr() == att.q_proj.weight.data_ptr() + att.q_proj.weight.numel() * 4
    assert torch.equal(model(ids)["logits"], before)
    model(ids)["logits"].sum().backward()
    assert flat.grad.abs().sum() > 0 and att.q_proj.weight.grad.data_ptr() == att.q_proj.weight.main_grad.data_ptr()


# ---- encoder ----
def _enc_cfg(**kw):
    base = dict(vocab_size=300, dim=32, n_layers=2, norm_eps=1e-5, dim_ffn=64, max_len=64, rope_theta=1e4, n_heads=4,
                n_kv_heads=2, model_type="embedding")
    base.update(kw)
    return EncoderConfig(**base)


@pytest.mark.parametrize("pooling", ["mean", "cls", "last"])
def test_encoder_pooling(pooling):
    enc = EmbeddingEncoder(_enc_cfg(pooling_type=pooling, normalize_embeddings=True)).eval()
    ids = torch.randint(0, 300, (3, 10))
    mask = torch.ones(3, 10, dtype=torch.bool)
    mask[2, 6:] = False
    out = enc(ids, input_mask=mask)
    assert out.shape == (3, 32) and torch.allclose(out.norm(dim=-1), torch.ones(3), atol=1e-5)
    assert enc(ids).shape == (3, 32)


def test_encoder_is_bidirectional_and_registered(tmp_path):
    assert AutoModel.is_registered("embedding") and AutoModel.is_registered("autoregressive_lm")
    enc = EmbeddingEncoder(_enc_cfg(pooling_type="cls")).eval()
    ids = torch.randint(0, 300, (1, 8))
    ids2 = ids.clone()
    ids2[0, 7] = (ids2[0, 7] + 5) % 300
    assert not torch.allclose(enc(ids), enc(ids2))  # the first position sees the last one
    lm = AutoRegressiveLM(tiny_config())
    enc.load_state_dict(lm.state_dict(), strict=True)  # lm_head.weight is dropped
    enc.save_pretrained(str(tmp_path / "enc"))
    assert isinstance(AutoModel.from_pretrained(str(tmp_path / "enc")), EmbeddingEncoder)


# ---- LoRA ----
def test_lora_linear_properties():
    base = Linear(16, 24)
    lora = LoRALinear(base, r=4, alpha=8)
    assert lora.weight is base.weight and not lora.weight.requires_grad
    assert lora.lora_A.shape == (4, 16) and lora.lora_B.shape == (24, 4) and lora.scaling == 2.0
    x = torch.randn(3, 16)
    assert torch.allclose(lora(x), base(x))  # B starts at zero
    lora.lora_B.data.normal_()
    want = lora(x)
    lora.merge()
    assert torch.allclose(lora(x), want, atol=1e-5) and not hasattr(lora, "lora_A")


def test_lora_inject_merge_save_load(tmp_path, caplog):
    model = AutoRegressiveLM(tiny_config()).eval()
    ids = torch.randint(0, 300, (2, 7))
    before = model(ids)["logits"]
    cfg = inject_lora(model, r=4, alpha=8)
    assert isinstance(cfg, LoRAConfig) and set(cfg.target_modules) == {"q_proj", "k_proj", "v_proj", "o_proj"}
    assert torch.allclose(model(ids)["logits"], before, atol=1e-6)
    keys = set(model.state_dict())
    assert {"layers.0.attention.q_proj.weight", "layers.0.attention.q_proj.lora_A",
            "layers.0.attention.q_proj.lora_B"} <= keys
    n = sum(isinstance(m, LoRALinear) for m in model.modules())
    inject_lora(model, r=4, alpha=8)  # repeated injection is a no-op
    assert sum(isinstance(m, LoRALinear) for m in model.modules()) == n
    inject_lora(model, r=4, alpha=8, target_modules={"up"})
    assert sum(isinstance(m, LoRALinear) for m in model.modules()) == n + 2
    trainable = [k for k, p in model.named_parameters() if p.requires_grad]
    assert all("lora_" in k or "norm" in k or "embed" in k or "lm_head" in k or ".gate." in k or ".down." in k
               for k in trainable)
    for m in model.modules():
        if isinstance(m, LoRALinear):
            m.lora_B.data.normal_(std=0.02)
    tuned = model(ids)["logits"]
    save_lora(model, str(tmp_path / "adapter"), LoRAConfig(r=4, alpha=8, target_modules=("q_proj", "k_proj", "v_proj", "o_proj", "up")))
    fresh = AutoRegressiveLM(tiny_config()).eval()
    fresh.load_state_dict({k: v for k, v in model.state_dict().items() if "lora_" not in k})
    load_lora(fresh, str(tmp_path / "adapter"))
    assert torch.allclose(fresh(ids)["logits"], tuned, atol=1e-5)
    merge_lora(model)
    assert torch.allclose(model(ids)["logits"], tuned, atol=1e-4)
    with pytest.raises(RuntimeError, match="No LoRA parameters"):
        save_lora(model, str(tmp_path / "x"), cfg)
    with caplog.at_level(logging.WARNING):
        merge_lora(AutoRegressiveLM(tiny_config()))
        inject_lora(AutoRegressiveLM(tiny_config()), target_modules={"nope"})
    assert "No LoRA layers to merge" in caplog.text and "No LoRA layers injected" in caplog.text


def test_lora_rank_mismatch(tmp_path):
    a = AutoRegressiveLM(tiny_config())
    inject_lora(a, r=4, alpha=8)
    save_lora(a, str(tmp_path / "ad"), LoRAConfig(r=4, alpha=8, target_modules=("q_proj",)))
    b = AutoRegressiveLM(tiny_config())
    inject_lora(b, r=2, alpha=8)
    with pytest.raises(RuntimeError, match="size mismatch"):
        load_lora(b, str(tmp_path / "ad"))


def test_int8_weight_only_model_close_to_full_precision():
    from khaosz_b200.ops.quant import Int8Linear, quantize_model_int8

    torch.manual_seed(0)
    model = AutoRegressiveLM(tiny_config()).eval()
    ids = torch.randint(0, 300, (2, 12))
    ref = model(ids)["logits"]
    n = quantize_model_int8(model)
    assert n == 2 * 7 and isinstance(model.layers[0].attention.q_proj, Int8Linear)
    got = model(ids)["logits"]
    assert (got - ref).abs().max().item() < 0.05 * ref.abs().max().item() + 0.02


def test_int8_packed_projections_match_separate_ones():
    from khaosz_b200.ops.quant import Int8Linear, int8_multi_linear, quantize_model_int8

    torch.manual_seed(0)
    model = AutoRegressiveLM(tiny_config()).eval()
    ids = torch.randint(0, 300, (2, 9))
    quantize_model_int8(model)
    att = model.layers[0].attention
    x = torch.randn(2, 9, 32)
    packed = int8_multi_linear(x, (att.q_proj, att.k_proj, att.v_proj))
    assert packed is not None and isinstance(att.q_proj, Int8Linear)
    assert torch.allclose(packed, torch.cat([att.q_proj(x), att.k_proj(x), att.v_proj(x)], -1), atol=1e-5)
    assert torch.isfinite(model(ids)["logits"]).all()


def test_server_loader_merges_lora_adapters(tmp_path, tokenizer_dir):
    """Adapters given to the server are folded into the base weights; the wrappers are gone afterwards."""
    import shutil

    from khaosz_b200.inference.api.server import _load
    from khaosz_b200.models.components.layers import Linear
    from khaosz_b200.models.components.lora import LoRAConfig, LoRALinear, inject_lora, save_lora

    torch.manual_seed(0)
    model = AutoRegressiveLM(tiny_config()).eval()
    params, adapter = tmp_path / "params", tmp_path / "adapter"
    model.save_pretrained(str(params))
    for name in os.listdir(tokenizer_dir):
        shutil.copy(os.path.join(tokenizer_dir, name), params / name)
    inject_lora(model, r=4, alpha=8, target_modules={"q_proj", "o_proj", "down"})
    with torch.no_grad():
        for m in model.modules():
            if isinstance(m, LoRALinear):
                m.lora_B.normal_(0, 0.05)
    save_lora(model, str(adapter), LoRAConfig(r=4, alpha=8, target_modules=("q_proj", "o_proj", "down")))
    ids = torch.randint(0, 300, (2, 9))
    with torch.no_grad():
        want = model(ids)["logits"]
    served, _ = _load(params, "cpu", torch.float32, adapter_path=adapter)
    assert not any(isinstance(m, LoRALinear) for m in served.modules())
    assert type(served.layers[0].attention.q_proj) is Linear
    with torch.no_grad():
        got = served(ids)["logits"]
        plain = _load(params, "cpu", torch.float32)[0](ids)["logits"]
    assert torch.allclose(got, want, atol=1e-5) and not torch.allclose(plain, want, atol=1e-3)
