"""Case-by-case behaviour of the LoRA adapters and the embedding encoder (the behaviours the
reference pins in ``tests/module/test_lora.py`` and ``tests/module/test_encoder.py``)."""
import json
import logging

import pytest
import torch

from conftest import tiny_config
from khaosz_b200 import AutoModel, AutoRegressiveLM, EncoderConfig
from khaosz_b200.models import EmbeddingEncoder, LoRAConfig, LoRALinear, inject_lora, load_lora, merge_lora, save_lora
from khaosz_b200.models.components.layers import Linear
from khaosz_b200.serialization import load_state_dict


def _wrapped(model):
    return sorted(name for name, m in model.named_modules() if isinstance(m, LoRALinear))


# ---- LoRALinear -------------------------------------------------------------------------------
def test_adapter_shares_and_freezes_the_base_weight():
    base = Linear(16, 24)
    lora = LoRALinear(base, r=4, alpha=8)
    assert lora.weight is base.weight and not lora.weight.requires_grad
    assert lora.lora_A.shape == (4, 16) and lora.lora_B.shape == (24, 4)
    assert lora.lora_A.requires_grad and lora.lora_B.requires_grad
    assert lora.scaling == 2.0 and lora.r == 4 and float(lora.lora_B.detach().abs().sum()) == 0.0
    assert lora.lora_A.dtype == base.weight.dtype and lora.lora_A.device == base.weight.device


def test_adapter_starts_as_the_identity_change():
    base = Linear(16, 24)
    lora = LoRALinear(base, r=4, alpha=8)
    x = torch.randn(5, 16)
    assert torch.equal(lora(x), base(x))


def test_adapter_adds_the_scaled_low_rank_product():
    base = Linear(16, 24)
    lora = LoRALinear(base, r=4, alpha=8)
    with torch.no_grad():
        lora.lora_B.normal_()
    x = torch.randn(5, 16)
    want = x @ base.weight.t() + (x @ lora.lora_A.t()) @ lora.lora_B.t() * 2.0
    assert torch.allclose(lora(x), want, atol=1e-5) and not torch.allclose(lora(x), base(x))


def test_adapter_passes_gradients_to_a_and_b_only():
    lora = LoRALinear(Linear(8, 8), r=2, alpha=2)
    with torch.no_grad():
        lora.lora_B.normal_()
    lora(torch.randn(3, 8)).sum().backward()
    assert lora.lora_A.grad is not None and lora.lora_B.grad is not None and lora.weight.grad is None


def test_merge_folds_the_adapter_into_the_weight_once():
    base = Linear(16, 24)
    lora = LoRALinear(base, r=4, alpha=8)
    with torch.no_grad():
        lora.lora_B.normal_()
    x = torch.randn(5, 16)
    want = lora(x)
    before = base.weight.detach().clone()
    lora.merge()
    assert not torch.equal(base.weight, before) and torch.allclose(lora(x), want, atol=1e-5)
    assert not hasattr(lora, "lora_A") and not hasattr(lora, "lora_B")
    merged = base.weight.detach().clone()
    lora.merge()                                        # a second merge changes nothing
    assert torch.equal(base.weight, merged)


# ---- injection --------------------------------------------------------------------------------
def test_default_targets_are_the_attention_projections():
    model = AutoRegressiveLM(tiny_config())
    cfg = inject_lora(model, r=4, alpha=8)
    assert isinstance(cfg, LoRAConfig) and (cfg.r, cfg.alpha) == (4, 8)
    assert set(cfg.target_modules) == {"q_proj", "k_proj", "v_proj", "o_proj"}
    assert _wrapped(model) == sorted(f"layers.{i}.attention.{p}" for i in range(2) for p in ("q_proj", "k_proj", "v_proj", "o_proj"))


def test_feed_forward_targets():
    model = AutoRegressiveLM(tiny_config())
    inject_lora(model, r=2, alpha=4, target_modules={"up", "gate", "down"})
    assert _wrapped(model) == sorted(f"layers.{i}.mlp.{p}" for i in range(2) for p in ("up", "gate", "down"))


def test_unknown_targets_inject_nothing_and_warn(caplog):
    model = AutoRegressiveLM(tiny_config())
    with caplog.at_level(logging.WARNING):
        inject_lora(model, target_modules={"no_such_layer"})
    assert _wrapped(model) == [] and "No LoRA layers injected" in caplog.text and "q_proj" in caplog.text


def test_injection_keeps_the_outputs():
    model = AutoRegressiveLM(tiny_config()).eval()
    ids = torch.randint(0, 300, (2, 7))
    before = model(ids)["logits"]
    inject_lora(model, r=4, alpha=8)
    assert torch.allclose(model(ids)["logits"], before, atol=1e-6)


def test_injecting_twice_wraps_nothing_twice_and_new_targets_are_added():
    model = AutoRegressiveLM(tiny_config())
    inject_lora(model, r=4, alpha=8, target_modules={"q_proj"})
    first = model.layers[0].attention.q_proj
    inject_lora(model, r=4, alpha=8, target_modules={"q_proj"})
    assert model.layers[0].attention.q_proj is first and len(_wrapped(model)) == 2
    inject_lora(model, r=4, alpha=8, target_modules={"q_proj", "v_proj"})
    assert len(_wrapped(model)) == 4 and model.layers[0].attention.q_proj is first


@pytest.mark.parametrize("extra,expected", [
    (dict(attn_type="mla", kv_lora_rank=8, qk_nope_head_dim=4, qk_rope_head_dim=4), ["kv_a_proj", "kv_b_proj", "o_proj", "q_proj"]),
    (dict(ffn_type="moe", n_routed_experts=2, n_shared_experts=1, n_activated_experts=1), ["down", "gate", "up"]),
])
def test_injection_into_the_other_architectures(extra, expected):
    model = AutoRegressiveLM(tiny_config(**extra)).eval()
    ids = torch.randint(0, 300, (1, 6))
    before = model(ids)["logits"]
    inject_lora(model, r=2, alpha=4, target_modules=set(expected))
    leaves = sorted({name.rpartition(".")[2] for name in _wrapped(model)})
    assert leaves == expected and torch.allclose(model(ids)["logits"], before, atol=1e-6)
    if "ffn_type" in extra:                             # every expert's projections, shared ones included
        assert sum("routed_experts" in n for n in _wrapped(model)) == 2 * 2 * 3
        assert sum("shared_experts" in n for n in _wrapped(model)) == 2 * 1 * 3


def test_state_dict_keys_of_a_wrapped_layer():
    model = AutoRegressiveLM(tiny_config())
    plain = set(model.state_dict())
    inject_lora(model, r=4, alpha=8, target_modules={"q_proj"})
    keys = set(model.state_dict())
    assert keys - plain == {f"layers.{i}.attention.q_proj.lora_{ab}" for i in range(2) for ab in "AB"}
    assert plain <= keys                                # the base names do not move


def test_base_weights_of_wrapped_layers_are_the_only_ones_frozen():
    model = AutoRegressiveLM(tiny_config())
    inject_lora(model, r=4, alpha=8, target_modules={"q_proj", "v_proj"})
    frozen = sorted(n for n, p in model.named_parameters() if not p.requires_grad)
    assert frozen == sorted(f"layers.{i}.attention.{p}.weight" for i in range(2) for p in ("q_proj", "v_proj"))


def test_wrapped_model_still_loads_a_plain_state_dict():
    src = AutoRegressiveLM(tiny_config())
    dst = AutoRegressiveLM(tiny_config())
    inject_lora(dst, r=4, alpha=8)
    missing, unexpected = dst.load_state_dict(src.state_dict(), strict=False)
    assert unexpected == [] and all("lora_" in k for k in missing)
    assert torch.equal(dst.layers[0].attention.q_proj.weight, src.layers[0].attention.q_proj.weight)


# ---- save / load / merge ------------------------------------------------------------------------
def test_adapter_files_and_round_trip(tmp_path):
    model = AutoRegressiveLM(tiny_config()).eval()
    cfg = inject_lora(model, r=4, alpha=8, target_modules={"q_proj", "down"})
    with torch.no_grad():
        for m in model.modules():
            if isinstance(m, LoRALinear):
                m.lora_B.normal_(std=0.05)
    save_lora(model, str(tmp_path / "ad"), cfg)
    assert sorted(p.name for p in (tmp_path / "ad").iterdir()) == ["adapter_config.json", "adapter_model.safetensors"]
    raw = json.loads((tmp_path / "ad" / "adapter_config.json").read_text())
    assert raw["r"] == 4 and raw["alpha"] == 8 and sorted(raw["target_modules"]) == ["down", "q_proj"]
    saved = load_state_dict(tmp_path / "ad" / "adapter_model.safetensors")
    assert all(k.endswith(("lora_A", "lora_B")) for k in saved) and len(saved) == 2 * 2 * 2

    ids = torch.randint(0, 300, (2, 7))
    fresh = AutoRegressiveLM(tiny_config()).eval()
    fresh.load_state_dict({k: v for k, v in model.state_dict().items() if "lora_" not in k})
    loaded = load_lora(fresh, str(tmp_path / "ad"))           # injects by the saved config, then loads
    assert (loaded.r, loaded.alpha) == (4, 8) and _wrapped(fresh) == _wrapped(model)
    assert torch.allclose(fresh(ids)["logits"], model(ids)["logits"], atol=1e-6)


def test_loading_onto_an_already_wrapped_model_reuses_its_layers(tmp_path, caplog):
    a = AutoRegressiveLM(tiny_config())
    cfg = inject_lora(a, r=4, alpha=8, target_modules={"q_proj"})
    with torch.no_grad():
        a.layers[0].attention.q_proj.lora_B.fill_(0.5)
    save_lora(a, str(tmp_path / "ad"), cfg)
    b = AutoRegressiveLM(tiny_config())
    inject_lora(b, r=4, alpha=8, target_modules={"q_proj"})
    layer = b.layers[0].attention.q_proj
    with caplog.at_level(logging.WARNING):
        load_lora(b, str(tmp_path / "ad"))
    assert b.layers[0].attention.q_proj is layer and float(layer.lora_B.detach().mean()) == 0.5
    assert "already has LoRA layers" in caplog.text


def test_loading_adapters_of_another_rank_fails_clearly(tmp_path):
    a = AutoRegressiveLM(tiny_config())
    cfg = inject_lora(a, r=4, alpha=8, target_modules={"q_proj"})
    save_lora(a, str(tmp_path / "ad"), cfg)
    b = AutoRegressiveLM(tiny_config())
    inject_lora(b, r=2, alpha=8, target_modules={"q_proj"})
    with pytest.raises(RuntimeError, match="size mismatch"):
        load_lora(b, str(tmp_path / "ad"))


def test_saving_without_adapters_fails(tmp_path):
    with pytest.raises(RuntimeError, match="No LoRA parameters"):
        save_lora(AutoRegressiveLM(tiny_config()), str(tmp_path / "x"), LoRAConfig())
    model = AutoRegressiveLM(tiny_config())
    cfg = inject_lora(model, r=2, alpha=4)
    merge_lora(model)
    with pytest.raises(RuntimeError, match="No LoRA parameters"):
        save_lora(model, str(tmp_path / "y"), cfg)


def test_merging_the_model_keeps_its_outputs_and_can_unwrap():
    model = AutoRegressiveLM(tiny_config()).eval()
    inject_lora(model, r=4, alpha=8)
    with torch.no_grad():
        for m in model.modules():
            if isinstance(m, LoRALinear):
                m.lora_B.normal_(std=0.05)
    ids = torch.randint(0, 300, (2, 7))
    want = model(ids)["logits"]
    merge_lora(model)
    assert torch.allclose(model(ids)["logits"], want, atol=1e-5) and len(_wrapped(model)) == 8
    assert not any("lora_" in k for k in model.state_dict())
    merge_lora(model, unwrap=True)
    assert _wrapped(model) == [] and type(model.layers[0].attention.q_proj) is Linear
    assert torch.allclose(model(ids)["logits"], want, atol=1e-5)


def test_merging_a_model_without_adapters_warns(caplog):
    with caplog.at_level(logging.WARNING):
        merge_lora(AutoRegressiveLM(tiny_config()))
    assert "No LoRA layers to merge" in caplog.text


# ---- encoder ----------------------------------------------------------------------------------
def _enc(**kw):
    base = dict(vocab_size=300, dim=32, n_layers=2, norm_eps=1e-5, dim_ffn=64, max_len=64, rope_theta=1e4, n_heads=4,
                n_kv_heads=2, model_type="embedding")
    base.update(kw)
    torch.manual_seed(0)
    return EmbeddingEncoder(EncoderConfig(**base)).eval()


def _hidden(enc, ids, mask=None):
    x = enc.embed_tokens(ids)
    rotary = enc.rotary_embedding(x, None)
    m = enc._mask(x, mask)
    for layer in enc.layers:
        x = layer(x, rotary, m, None, causal=False)
    return enc.norm(x)


def test_mean_pooling_averages_all_positions():
    enc = _enc(pooling_type="mean")
    ids = torch.randint(0, 300, (2, 9))
    assert torch.allclose(enc(ids), _hidden(enc, ids).mean(dim=1), atol=1e-6) and enc(ids).shape == (2, 32)


def test_cls_pooling_takes_the_first_position_and_last_pooling_the_last():
    ids = torch.randint(0, 300, (2, 9))
    enc = _enc(pooling_type="cls")
    assert torch.allclose(enc(ids), _hidden(enc, ids)[:, 0], atol=1e-6)
    enc = _enc(pooling_type="last")
    assert torch.allclose(enc(ids), _hidden(enc, ids)[:, -1], atol=1e-6)


def test_padding_is_ignored_by_attention_and_pooling():
    ids = torch.randint(0, 300, (1, 6))
    padded = torch.cat([ids, torch.randint(0, 300, (1, 4))], dim=1)
    mask = torch.tensor([[True] * 6 + [False] * 4])
    for pooling in ("mean", "last", "cls"):
        enc = _enc(pooling_type=pooling)
        assert torch.allclose(enc(padded, input_mask=mask), enc(ids), atol=1e-5), pooling


def test_default_pooling_is_mean_without_normalisation():
    enc = _enc()
    assert enc.pooling_type == "mean" and not enc.normalize_embeddings
    out = enc(torch.randint(0, 300, (3, 5)))
    assert not torch.allclose(out.norm(dim=-1), torch.ones(3), atol=1e-3)


def test_normalised_embeddings_have_unit_length():
    out = _enc(normalize_embeddings=True)(torch.randint(0, 300, (4, 5)))
    assert torch.allclose(out.norm(dim=-1), torch.ones(4), atol=1e-5)


def test_encoder_sees_both_directions():
    enc = _enc(pooling_type="cls")
    ids = torch.randint(0, 300, (1, 8))
    other = ids.clone()
    other[0, -1] = (other[0, -1] + 7) % 300
    assert not torch.allclose(enc(ids), enc(other))


def test_encoder_is_registered_with_automodel():
    assert AutoModel.is_registered("embedding") and AutoModel.is_registered("autoregressive_lm")
    assert not AutoModel.is_registered("diffusion")


def test_encoder_takes_a_language_model_checkpoint():
    lm = AutoRegressiveLM(tiny_config())
    enc = _enc()
    assert "lm_head.weight" in lm.state_dict()
    enc.load_state_dict(lm.state_dict(), strict=True)          # the head is dropped, everything else must fit
    assert torch.equal(enc.embed_tokens.weight, lm.embed_tokens.weight)
    assert torch.equal(enc.layers[1].mlp.down.weight, lm.layers[1].mlp.down.weight)


def test_encoder_save_and_load(tmp_path):
    enc = _enc(pooling_type="last", normalize_embeddings=True)
    enc.save_pretrained(str(tmp_path / "enc"))
    assert json.loads((tmp_path / "enc" / "config.json").read_text())["model_type"] == "embedding"
    back = AutoModel.from_pretrained(str(tmp_path / "enc")).eval()
    assert isinstance(back, EmbeddingEncoder) and back.pooling_type == "last" and back.normalize_embeddings
    ids = torch.randint(0, 300, (2, 6))
    assert torch.allclose(back(ids), enc(ids), atol=1e-6)
