"""Block-granular full sharding (``fsdp_block``) on CPU: one process and gloo ranks against the dense /
data-parallel result, slot reuse over more than two blocks, accumulation, checkpoints, recompute, MoE."""
import pytest
import torch
import torch.distributed as dist

from khaosz_b200.parallel import ExecutorFactory, spawn_parallel_fn


def _model(layers=5, moe=False, tie=True, seed=11, mla=False):
    from khaosz_b200 import AutoRegressiveLM, AutoRegressiveLMConfig

    ffn = dict(ffn_type="moe", n_routed_experts=4, n_shared_experts=1, n_activated_experts=2) if moe else {}
    att = dict(attn_type="mla", kv_lora_rank=16, qk_nope_head_dim=8, qk_rope_head_dim=8, use_qk_norm=True,
               use_gated_attention=True) if mla else {}
    cfg = AutoRegressiveLMConfig(vocab_size=300, dim=64, n_layers=layers, norm_eps=1e-5, dim_ffn=96, tie_weight=tie,
                                 max_len=64, rope_theta=1e4, n_heads=4, n_kv_heads=2, **ffn, **att)
    torch.manual_seed(seed)
    m = AutoRegressiveLM(cfg)
    with torch.no_grad():
        for name, p in m.named_parameters():
            if "norm" in name:
                p.add_(0.1 * torch.randn_like(p))
    return m


def _train(mode, rank, world, steps=3, accum=2, recompute=False, **model_kw):
    from khaosz_b200.trainer import FusedAdamW, StrategyFactory

    model = _model(**model_kw)
    ex = ExecutorFactory.create(mode, grad_accum_steps=accum)
    opt = FusedAdamW(model.parameters(), lr=1e-3, betas=(0.9, 0.95), weight_decay=0.01)
    model, opt, _, _ = ex.prepare(model, opt, None, None)
    if recompute:
        from khaosz_b200.models.components.block import DecoderBlock
        from khaosz_b200.trainer.callbacks import GradientCheckpointingCallback

        cb = GradientCheckpointingCallback([DecoderBlock])
        model.apply(cb._enable)
    strat = StrategyFactory.create("seq", model, "cpu")
    data = torch.randint(0, 300, (steps * accum, 2 * world, 33), generator=torch.Generator().manual_seed(5))
    losses = []
    for i in range(steps * accum):
        mine = data[i, 2 * rank:2 * rank + 2]
        with ex.accumulate(model):
            loss = strat({"input_ids": mine[:, :-1], "target_ids": mine[:, 1:]})
            ex.backward(loss / accum)
            if ex.sync_gradients:
                opt.fused_clip(1.0)
                opt.step()
                opt.zero_grad()
        losses.append(loss.item())
    return model, ex, opt, losses


def test_one_process_equals_the_dense_run():
    dense, ex0, opt0, l0 = _train("none", 0, 1)
    model, ex, opt, l1 = _train("fsdp_block", 0, 1)
    assert l1 == pytest.approx(l0, rel=1e-5, abs=1e-6)
    sd = ex.unwrap_model(model)
    for k, v in dense.state_dict().items():
        assert torch.allclose(sd[k], v, rtol=1e-5, atol=1e-6), k
    a, b = opt0.state_dict(), opt.state_dict()
    assert len(a["state"]) == len(b["state"])
    for i in a["state"]:
        assert torch.allclose(a["state"][i]["exp_avg"], b["state"][i]["exp_avg"], rtol=1e-5, atol=1e-8), i
    # five blocks went through two images: every backward re-gathered what the forward had displaced
    assert ex.units.gathers > 2 * 5 and ex.units.reductions == 3 * 2 * 5
    # outside its backward pass a block's parameters carry no gradient tensor; the replicated ones keep theirs
    assert all(p.grad is None for u in ex.units.units for p in u.params)
    assert all(p.grad is not None for p in ex.units.rest)


def _ranks_case(out, moe=False, recompute=False, tie=True, mla=False):
    rank, world = dist.get_rank(), dist.get_world_size()
    kw = dict(moe=moe, tie=tie, mla=mla)
    ref_model, ref_ex, ref_opt, ref_losses = _train("ddp", rank, world, **kw)
    model, ex, opt, losses = _train("fsdp_block", rank, world, recompute=recompute, **kw)
    assert losses == pytest.approx(ref_losses, rel=1e-4, abs=1e-5)
    sd = ex.unwrap_model(model)                       # collective, dense names
    ref_sd = ref_ex.unwrap_model(ref_model)
    assert list(sd) == list(ref_sd)
    for k, v in ref_sd.items():
        assert torch.allclose(sd[k], v, rtol=1e-4, atol=1e-5), k
    u = ex.units
    blocks = sum(x.numel for x in u.units)
    assert u.local_numel == blocks // world + u.rest_numel      # 1 / world of the block weights per rank
    assert u.data.numel() == u.local_numel and opt.optimizer._m.numel() == u.local_numel

    # optimizer state: dense layout out, this rank's pieces back in
    state, ref_state = opt.state_dict(), ref_opt.state_dict()
    for i in ref_state["state"]:
        assert torch.allclose(state["state"][i]["exp_avg"], ref_state["state"][i]["exp_avg"], rtol=1e-3, atol=1e-7), i
        assert state["state"][i]["exp_avg"].shape == ref_state["state"][i]["exp_avg"].shape
    if rank == 0:
        torch.save({"opt": state, "sd": sd}, out)
    dist.barrier()
    saved = torch.load(out, weights_only=False)
    model2, ex2, opt2, _ = _train("fsdp_block", rank, world, steps=0, **kw)
    ex2.units.load_full_state_dict(saved["sd"])
    opt2.load_state_dict(saved["opt"])
    assert torch.equal(ex2.units.data, u.data)
    assert torch.equal(opt2.optimizer._m, opt.optimizer._m) and torch.equal(opt2.optimizer._v, opt.optimizer._v)
    assert opt2.optimizer._step_count == opt.optimizer._step_count

    # a forward without gradients (validation) gathers on demand and sees the updated weights
    ids = torch.randint(0, 300, (2, 16), generator=torch.Generator().manual_seed(1))
    with torch.no_grad():
        got = model2(ids)["logits"]
    dense = _model(**kw)
    dense.load_state_dict(saved["sd"])
    with torch.no_grad():
        want = dense(ids)["logits"]
    assert torch.allclose(got, want, rtol=1e-4, atol=1e-5)
    dist.barrier()


@pytest.mark.parametrize("world,port,kw", [(2, "29741", {}), (4, "29742", {"tie": False}), (2, "29743", {"moe": True}),
                                           (2, "29744", {"recompute": True}), (2, "29746", {"mla": True})])
def test_ranks_match_data_parallel(world, port, kw, tmp_path):
    spawn_parallel_fn(_ranks_case, world_size=world, backend="gloo", master_addr="127.0.0.1", master_port=port,
                      out=str(tmp_path / "s.pt"), **kw)


def test_rejects_what_it_cannot_shard():
    from khaosz_b200.trainer import FusedAdamW

    model = _model(layers=2)
    next(model.layers[0].parameters()).requires_grad_(False)
    with pytest.raises(NotImplementedError):
        ExecutorFactory.create("fsdp_block").prepare(model, None, None, None)
    model = _model(layers=2)
    with pytest.raises(NotImplementedError):
        ExecutorFactory.create("fsdp_block").prepare(model, torch.optim.SGD(model.parameters(), lr=0.1), None, None)
    assert FusedAdamW is not None


# ---- DPO / GRPO: the frozen copy is sharded block by block like the policy ----
def _preference_case():
    from khaosz_b200.trainer import FusedAdamW, StrategyFactory

    rank, world = dist.get_rank(), dist.get_world_size()

    def run(mode):
        model = _model(layers=3)
        ex = ExecutorFactory.create(mode, grad_accum_steps=1)
        opt = FusedAdamW(model.parameters(), lr=1e-3)
        model, opt, _, _ = ex.prepare(model, opt, None, None)
        dpo = StrategyFactory.create("dpo", model, "cpu", executor=ex, model_fn=lambda: _model(layers=3), beta=0.1)
        g = torch.Generator().manual_seed(5 + rank)
        losses = []
        for _ in range(3):
            batch = {"chosen": torch.randint(0, 300, (2, 24), generator=g), "rejected": torch.randint(0, 300, (2, 24), generator=g),
                     "chosen_mask": torch.ones(2, 24, dtype=torch.bool), "rejected_mask": torch.ones(2, 24, dtype=torch.bool)}
            with ex.accumulate(model):
                losses.append(ex.micro_step(dpo, batch).item())
                opt.step()
                opt.zero_grad()
        return model, ex, dpo, losses

    _, ref_ex, ref_dpo, ref_losses = run("ddp")
    model, ex, dpo, losses = run("fsdp_block")
    assert losses == pytest.approx(ref_losses, rel=1e-4, abs=1e-5)
    assert losses[0] == pytest.approx(0.6931, abs=2e-3)           # policy == frozen copy before the first update
    assert getattr(ref_dpo.ref_model, "sharded_units", None) is None
    units = dpo.ref_model.sharded_units
    assert units.frozen and units.grad is None and not units.g_image
    assert units.data.numel() == sum(u.numel for u in units.units) // world + units.rest_numel
    assert not any(p.requires_grad for p in dpo.ref_model.parameters())

    # GRPO refreshes its old-policy copy from the (sharded) policy: every rank takes its pieces
    grpo = StrategyFactory.create("grpo", model, "cpu", executor=ex, model_fn=lambda: _model(layers=3), group_size=4,
                                  sync_interval=1)
    before = grpo.ref_model.sharded_units.data.clone()
    with torch.no_grad():
        ex.units.data.add_(0.01)                                  # the policy moves on
        ex.units.invalidate()
    grpo.sync_ref_model()
    assert torch.allclose(grpo.ref_model.sharded_units.data, before + 0.01, atol=1e-6)
    ids = torch.randint(0, 300, (2, 12), generator=torch.Generator().manual_seed(2))
    with torch.no_grad():
        assert torch.allclose(grpo.ref_model(ids)["logits"], model(ids)["logits"], rtol=1e-4, atol=1e-5)
    dist.barrier()


def test_frozen_copy_of_dpo_and_grpo_is_sharded_like_the_policy():
    spawn_parallel_fn(_preference_case, world_size=2, backend="gloo", master_addr="127.0.0.1", master_port="29745")


def test_fsdp_falls_back_to_resident_parameters_where_it_cannot_shard(caplog):
    from khaosz_b200.trainer import FusedAdamW

    model = _model(layers=2)
    next(model.layers[0].parameters()).requires_grad_(False)          # e.g. a base weight under LoRA
    ex = ExecutorFactory.create("fsdp")
    opt = FusedAdamW([p for p in model.parameters() if p.requires_grad], lr=1e-3)
    with caplog.at_level("WARNING"):
        ex.prepare(model, opt, None, None)
    assert ex.units is None and "frozen parameters" in caplog.text
    # asked for explicitly: no warning, no sharding
    model = _model(layers=2)
    ex = ExecutorFactory.create("fsdp", shard_parameters=False)
    ex.prepare(model, FusedAdamW(model.parameters(), lr=1e-3), None, None)
    assert ex.units is None
    # and the default shards
    model = _model(layers=2)
    ex = ExecutorFactory.create("fsdp")
    ex.prepare(model, FusedAdamW(model.parameters(), lr=1e-3), None, None)
    assert ex.units is not None and ex.flat is ex.units.flat


@pytest.mark.parametrize("prefetch", [True, False])
def test_two_forward_passes_before_one_backward(prefetch):
    """The images are re-gathered on demand in whatever order autograd visits the blocks: two forward
    passes, then one backward pass through both graphs, give the dense gradients."""
    from khaosz_b200.parallel.unit_shard import ShardedUnits

    dense, sharded = _model(layers=4), _model(layers=4)
    units = ShardedUnits(sharded, prefetch=prefetch)
    g = torch.Generator().manual_seed(9)
    a, b = torch.randint(0, 300, (2, 20), generator=g), torch.randint(0, 300, (2, 20), generator=g)
    (dense(a)["logits"].float().pow(2).mean() + dense(b)["logits"].float().pow(2).mean()).backward()
    (sharded(a)["logits"].float().pow(2).mean() + sharded(b)["logits"].float().pow(2).mean()).backward()
    units.finish_backward()
    grads = {}
    for u in units.units:      # one process owns every piece whole
        for p, o in zip(u.params, u.offsets):
            grads[id(p)] = units.grad[u.local + o:u.local + o + p.numel()].view(p.shape)
    for (name, pd), ps in zip(dense.named_parameters(), sharded.parameters()):
        got = grads.get(id(ps), ps.grad)
        assert torch.allclose(got, pd.grad, rtol=1e-4, atol=1e-6), name
    assert units.reductions == 2 * 4


def test_unit_layout_properties():
    """Offsets are 16-byte aligned and disjoint, the unit length divides by ``8 * ws`` for every world size, and
    the pieces of all ranks tile the unit exactly."""
    import random

    import torch.nn as nn

    from khaosz_b200.parallel.unit_shard import _Unit

    rng = random.Random(0)
    for _ in range(50):
        ws = rng.choice([1, 2, 3, 4, 8])
        params = [nn.Parameter(torch.empty(rng.randint(1, 9), rng.randint(1, 37))) for _ in range(rng.randint(1, 7))]
        u = _Unit(params, ws)
        end = 0
        for p, o in zip(u.params, u.offsets):
            assert o % 8 == 0 and o >= end
            end = o + p.numel()
        assert u.numel >= end and u.numel % (8 * ws) == 0 and u.numel - end < 8 * ws + 8
        assert u.per * ws == u.numel and u.per % 8 == 0
