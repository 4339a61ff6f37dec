"""The model's building blocks against their textbook formulas, written out with plain tensor
operations, plus the model-level contracts (tied weights, padding, state-dict names, file round trips).
Behaviour reference: ``astrai/model/components/*.py`` and ``astrai/model/transformer.py``."""
import json
import math

import pytest
import torch
import torch.nn.functional as F

from conftest import tiny_config
from khaosz_b200 import AutoModel, AutoRegressiveLM, AutoRegressiveLMConfig, ops
from khaosz_b200.models.components.attention import GQA, MLA
from khaosz_b200.models.components.block import DecoderBlock
from khaosz_b200.models.components.ffn import MLP, DeepSeekMoE
from khaosz_b200.models.components.layers import Embedding, Linear, RMSNorm, RotaryEmbedding, ntk_scaled_base
from khaosz_b200.serialization import (load_json, load_safetensors, load_torch, save_json, save_safetensors, save_torch)


# ---- layers -----------------------------------------------------------------------------------
def test_linear_is_bias_free_x_times_w_transposed():
    lin = Linear(6, 4)
    assert lin.weight.shape == (4, 6) and lin.bias is None and [n for n, _ in lin.named_parameters()] == ["weight"]
    x = torch.randn(3, 5, 6)
    assert torch.allclose(lin(x), x @ lin.weight.t(), atol=1e-6)
    res = torch.randn(3, 5, 4)
    assert torch.allclose(lin(x, res), x @ lin.weight.t() + res, atol=1e-6)            # residual epilogue


def test_linear_with_bias_and_init_range():
    lin = Linear(64, 32, bias=True)
    assert lin.bias.shape == (32,) and float(lin.bias.detach().abs().sum()) == 0.0
    bound = 1.0 / math.sqrt(64)                         # kaiming-uniform with a = sqrt(5)
    assert float(lin.weight.detach().abs().max()) <= bound + 1e-6 and float(lin.weight.detach().std()) > 0.3 * bound
    x = torch.randn(2, 64)
    with torch.no_grad():
        lin.bias.fill_(0.5)
    assert torch.allclose(lin(x), x @ lin.weight.t() + 0.5, atol=1e-6)


def test_embedding_looks_rows_up_and_starts_narrow():
    torch.manual_seed(0)
    emb = Embedding(500, 64)
    assert emb.weight.shape == (500, 64) and abs(float(emb.weight.detach().std()) - 0.02) < 0.002
    ids = torch.tensor([[1, 499], [0, 1]])
    assert torch.equal(emb(ids), emb.weight[ids])


def test_rmsnorm_formula():
    norm = RMSNorm(16, 1e-5)
    assert torch.equal(norm.weight, torch.ones(16))
    with torch.no_grad():
        norm.weight.uniform_(0.5, 1.5)
    x = torch.randn(3, 7, 16) * 4
    want = x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + 1e-5) * norm.weight
    assert torch.allclose(norm(x), want, atol=1e-5)
    y, passthrough = norm.fork(x)
    assert torch.allclose(y, want, atol=1e-5) and torch.equal(passthrough, x)


def test_rope_rotates_interleaved_pairs_like_complex_multiplication():
    rot = RotaryEmbedding(8, 32, base=10000.0)
    x = torch.randn(2, 5, 3, 8)
    cs, pos = rot(x)
    assert cs.shape == (32, 4, 2) and cs.dtype == torch.float32 and pos is None
    inv = 1.0 / (10000.0 ** (torch.arange(0, 8, 2, dtype=torch.float64) / 8))
    ang = torch.outer(torch.arange(5, dtype=torch.float64), inv)
    unit = torch.polar(torch.ones_like(ang), ang)                                   # e^{i * position * frequency}
    want = torch.view_as_real(torch.view_as_complex(x.double().reshape(2, 5, 3, 4, 2)) * unit[None, :, None, :])
    assert torch.allclose(ops.rope(x, cs, pos), want.reshape(2, 5, 3, 8).float(), atol=1e-5)
    assert torch.allclose(ops.rope(x, cs, pos)[:, 0], x[:, 0], atol=1e-6)           # position 0 is the identity


def test_rope_with_explicit_positions_and_norm_preservation():
    rot = RotaryEmbedding(8, 32)
    x = torch.randn(2, 4, 2, 8)
    cs, _ = rot(x)
    pos = torch.tensor([[3, 4, 5, 6], [0, 9, 1, 30]])
    out = ops.rope(x, cs, pos)
    full = ops.rope(torch.randn(2, 31, 2, 8).index_copy(1, torch.tensor([3, 4, 5, 6]), x[:1].expand(2, -1, -1, -1)), cs, None)
    assert torch.allclose(out[0], full[0, 3:7], atol=1e-6)                          # same as sitting at those positions
    assert torch.allclose(out.norm(dim=-1), x.norm(dim=-1), atol=1e-5)              # a rotation keeps lengths


def test_rope_scores_depend_on_relative_position_only():
    rot = RotaryEmbedding(16, 64)
    q, k = torch.randn(1, 1, 1, 16), torch.randn(1, 1, 1, 16)
    cs, _ = rot(q)

    def score(pq, pk):
        return float((ops.rope(q, cs, torch.tensor([[pq]])) * ops.rope(k, cs, torch.tensor([[pk]]))).sum())

    assert score(5, 2) == pytest.approx(score(25, 22), abs=1e-4) and score(5, 2) != pytest.approx(score(5, 3), abs=1e-4)


def test_ntk_scaling_raises_the_base():
    assert ntk_scaled_base(10000.0, 1.0, 64) == 10000.0
    assert ntk_scaled_base(10000.0, 4.0, 64) == pytest.approx(10000.0 * 4.0 ** (64 / 62))
    scaled = RotaryEmbedding(64, 16, 10000.0, {"type": "ntk", "factor": 4.0})
    plain = RotaryEmbedding(64, 16, 10000.0)
    assert scaled.base > plain.base and not torch.allclose(scaled.cos_sin, plain.cos_sin)
    assert "cos_sin" not in scaled.state_dict()                                     # a buffer that is not saved


# ---- feed-forward -----------------------------------------------------------------------------
def test_swiglu_mlp_formula():
    mlp = MLP(16, 40)
    assert sorted(n for n, _ in mlp.named_parameters()) == ["down.weight", "gate.weight", "up.weight"]
    x = torch.randn(2, 5, 16)
    want = (F.silu(x @ mlp.gate.weight.t()) * (x @ mlp.up.weight.t())) @ mlp.down.weight.t()
    assert torch.allclose(mlp(x), want, atol=1e-5)
    res = torch.randn(2, 5, 16)
    assert torch.allclose(mlp(x, res), want + res, atol=1e-5)


def test_moe_matches_a_per_token_loop():
    torch.manual_seed(0)
    moe = DeepSeekMoE(16, 24, n_routed_experts=4, n_shared_experts=2, n_activated_experts=2).eval()
    x = torch.randn(2, 6, 16)
    flat = x.reshape(-1, 16)
    probs = torch.softmax(flat @ moe.router.weight.t(), dim=-1)
    want = torch.zeros_like(flat)
    for t in range(flat.shape[0]):
        w, idx = torch.topk(probs[t], 2)
        w = w / w.sum()
        for weight, e in zip(w, idx):
            want[t] += weight * moe.routed_experts[int(e)](flat[t:t + 1])[0]
        want[t] += sum(e(flat[t:t + 1])[0] for e in moe.shared_experts) / 2
    assert torch.allclose(moe(x), want.view(2, 6, 16), atol=1e-5)


def test_moe_routing_weights_are_renormalised_and_experts_train():
    moe = DeepSeekMoE(8, 12, n_routed_experts=3, n_shared_experts=0, n_activated_experts=2)
    w, idx = moe.route(torch.randn(10, 8))
    assert w.shape == idx.shape == (10, 2) and torch.allclose(w.sum(-1), torch.ones(10), atol=1e-6)
    assert int(idx.max()) < 3 and (idx[:, 0] != idx[:, 1]).all()
    moe(torch.randn(4, 5, 8)).sum().backward()
    assert moe.router.weight.grad is not None and any(e.up.weight.grad is not None for e in moe.routed_experts)
    keys = set(moe.state_dict())
    assert "router.weight" in keys and "routed_experts.2.down.weight" in keys and not any("shared" in k for k in keys)


# ---- attention --------------------------------------------------------------------------------
def _manual_gqa(attn, x, cs):
    B, S, _ = x.shape
    H, Hkv, D = attn.n_heads, attn.n_kv_heads, attn.head_dim
    q = ops.rope((x @ attn.q_proj.weight.t()).view(B, S, H, D), cs, None)
    k = ops.rope((x @ attn.k_proj.weight.t()).view(B, S, Hkv, D), cs, None)
    v = (x @ attn.v_proj.weight.t()).view(B, S, Hkv, D)
    if attn.use_qk_norm:
        q, k = attn.q_norm(q), attn.k_norm(k)
    k, v = k.repeat_interleave(H // Hkv, dim=2), v.repeat_interleave(H // Hkv, dim=2)      # one KV head per query head
    scores = torch.einsum("bshd,bthd->bhst", q, k) / math.sqrt(D)
    scores = scores.masked_fill(torch.ones(S, S, dtype=torch.bool).triu(1), float("-inf"))
    ctx = torch.einsum("bhst,bthd->bshd", scores.softmax(-1), v).reshape(B, S, H * D)
    if attn.use_gated_attention:
        ctx = ctx * torch.sigmoid(x @ attn.gate.weight.t())
    return ctx @ attn.o_proj.weight.t()


@pytest.mark.parametrize("qk_norm,gated", [(False, False), (True, False), (False, True), (True, True)])
def test_grouped_query_attention_formula(qk_norm, gated):
    torch.manual_seed(0)
    attn = GQA(32, n_heads=4, n_kv_heads=2, use_qk_norm=qk_norm, norm_eps=1e-5, use_gated_attention=gated, layer_id=0)
    if qk_norm:
        with torch.no_grad():
            attn.q_norm.weight.uniform_(0.5, 1.5)
            attn.k_norm.weight.uniform_(0.5, 1.5)
    x = torch.randn(2, 7, 32)
    cs, _ = RotaryEmbedding(8, 16)(x)
    assert torch.allclose(attn(x, (cs, None)), _manual_gqa(attn, x, cs), atol=1e-5)
    names = sorted(n for n, _ in attn.named_parameters())
    assert ("gate.weight" in names) == gated and ("q_norm.weight" in names) == qk_norm


def test_attention_rejects_head_counts_that_do_not_divide():
    with pytest.raises(ValueError):
        GQA(30, n_heads=4, n_kv_heads=2, use_qk_norm=False, norm_eps=1e-5, use_gated_attention=False, layer_id=0)
    with pytest.raises(ValueError):
        GQA(32, n_heads=4, n_kv_heads=3, use_qk_norm=False, norm_eps=1e-5, use_gated_attention=False, layer_id=0)


def test_latent_attention_shapes_and_rotated_slice():
    torch.manual_seed(0)
    attn = MLA(32, n_heads=4, n_kv_heads=2, kv_lora_rank=8, qk_nope_head_dim=4, qk_rope_head_dim=4, norm_eps=1e-5,
               use_qk_norm=False, use_gated_attention=False, layer_id=0)
    assert attn.q_proj.weight.shape == (32, 32) and attn.kv_a_proj.weight.shape == (8, 32)
    assert attn.kv_b_proj.weight.shape == (2 * 2 * 8, 8) and attn.kv_norm.weight.shape == (8,)
    x = torch.randn(2, 6, 32)
    cs, _ = RotaryEmbedding(4, 16)(x)
    out = attn(x, (cs, None))
    assert out.shape == (2, 6, 32) and torch.isfinite(out).all()
    later = x.clone()
    later[:, -1] += 1.0
    assert torch.allclose(attn(later, (cs, None))[:, :-1], out[:, :-1], atol=1e-6)          # causal


def test_decoder_block_is_pre_norm_residual():
    torch.manual_seed(0)
    cfg = tiny_config()
    model = AutoRegressiveLM(cfg).eval()
    block = model.layers[0]
    assert isinstance(block, DecoderBlock)
    x = torch.randn(2, 5, cfg.dim)
    rotary = model.rotary_embedding(x, None)
    h = x + block.attention(block.input_norm(x), rotary)
    want = h + block.mlp(block.post_attention_norm(h))
    assert torch.allclose(block(x, rotary), want, atol=1e-5)


# ---- model-level contracts ----------------------------------------------------------------------
def test_logits_are_the_head_applied_to_the_normed_hidden_states():
    model = AutoRegressiveLM(tiny_config()).eval()
    out = model(torch.randint(0, 300, (2, 6)))
    assert set(out) == {"logits", "hidden_states"} and out["logits"].shape == (2, 6, 300)
    assert torch.allclose(out["logits"], out["hidden_states"] @ model.lm_head.weight.t(), atol=1e-5)


def test_padding_mask_without_positions_changes_nothing():
    model = AutoRegressiveLM(tiny_config()).eval()
    ids = torch.randint(0, 300, (2, 8))
    mask = torch.ones(2, 8, dtype=torch.bool)
    mask[1, 5:] = False
    assert torch.equal(model(ids, input_mask=mask)["logits"], model(ids)["logits"])
    out = model(ids, input_mask=mask, position_ids=torch.arange(8).expand(2, 8))["logits"]
    assert torch.isfinite(out).all() and torch.allclose(out[0], model(ids)["logits"][0], atol=1e-5)


@pytest.mark.parametrize("tied", [True, False])
def test_tied_and_untied_heads(tied, tmp_path):
    model = AutoRegressiveLM(tiny_config(tie_weight=tied))
    same = model.lm_head.weight.data_ptr() == model.embed_tokens.weight.data_ptr()
    assert same == tied and ("lm_head.weight" in model.state_dict()) == (not tied)
    n_params = sum(p.numel() for p in model.parameters())
    assert n_params == sum(p.numel() for p in AutoRegressiveLM(tiny_config(tie_weight=not tied)).parameters()) + \
        (-1 if tied else 1) * 300 * 32
    model.save_pretrained(str(tmp_path / "m"))
    back = AutoModel.from_pretrained(str(tmp_path / "m"))
    assert (back.lm_head.weight.data_ptr() == back.embed_tokens.weight.data_ptr()) == tied
    ids = torch.randint(0, 300, (1, 5))
    assert torch.allclose(back.eval()(ids)["logits"], model.eval()(ids)["logits"], atol=1e-6)


def test_untied_model_reads_a_tied_checkpoint_into_two_separate_tensors():
    tied = AutoRegressiveLM(tiny_config(tie_weight=True))
    untied = AutoRegressiveLM(tiny_config(tie_weight=False))
    untied.load_state_dict(tied.state_dict())
    assert torch.equal(untied.lm_head.weight, tied.embed_tokens.weight)
    assert untied.lm_head.weight.data_ptr() != untied.embed_tokens.weight.data_ptr()


def test_config_file_drops_unset_fields_and_dispatches_by_model_type(tmp_path):
    cfg = tiny_config()
    cfg.to_file(str(tmp_path / "config.json"))
    raw = json.loads((tmp_path / "config.json").read_text())
    assert "model_type" not in raw and "kv_lora_rank" not in raw and "rope_scaling" not in raw   # unset fields stay out
    back = AutoRegressiveLMConfig.from_file(str(tmp_path / "config.json"))
    assert back.to_dict() == cfg.to_dict()
    assert isinstance(AutoModel.from_pretrained(str(tmp_path)), AutoRegressiveLM)          # the default model type
    (tmp_path / "config.json").write_text(json.dumps({**raw, "model_type": "autoregressive_lm"}))
    assert isinstance(AutoModel.from_pretrained(str(tmp_path)), AutoRegressiveLM)
    (tmp_path / "config.json").write_text(json.dumps({**raw, "model_type": "nothing_known"}))
    with pytest.raises(ValueError):
        AutoModel.from_pretrained(str(tmp_path))


# ---- file helpers -------------------------------------------------------------------------------
def test_serialization_helpers_round_trip(tmp_path):
    tensors = {"a": torch.arange(6, dtype=torch.bfloat16).view(2, 3), "b.c": torch.randn(4)}
    save_safetensors(tensors, tmp_path / "t.safetensors")
    back = load_safetensors(tmp_path / "t.safetensors")
    assert set(back) == {"a", "b.c"} and back["a"].dtype == torch.bfloat16 and torch.equal(back["b.c"], tensors["b.c"])
    save_json({"x": 1, "y": [1, 2], "z": {"k": None}}, tmp_path / "d.json")
    assert load_json(tmp_path / "d.json") == {"x": 1, "y": [1, 2], "z": {"k": None}}
    save_torch({"step": 3, "t": torch.ones(2)}, tmp_path / "o.pt")
    obj = load_torch(tmp_path / "o.pt")
    assert obj["step"] == 3 and torch.equal(obj["t"], torch.ones(2))
