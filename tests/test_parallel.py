"""Process launch and executor parity on CPU (gloo, world size 2)."""
import os

import pytest
import torch
import torch.distributed as dist

from khaosz_b200.parallel import ExecutorFactory, only_on_rank, spawn_parallel_fn


def _allreduce(out_dir):
    t = torch.tensor([float(dist.get_rank() + 1)])
    dist.all_reduce(t)
    assert t.item() == 3.0

    @only_on_rank(0)
    def mark():
        open(os.path.join(out_dir, f"rank{dist.get_rank()}"), "w").close()
        return "done"

    assert mark() == ("done" if dist.get_rank() == 0 else None)


def test_spawn_gloo_default_device_type(tmp_path):
    spawn_parallel_fn(_allreduce, world_size=2, backend="gloo", master_addr="127.0.0.1", master_port="29621",
                      out_dir=str(tmp_path))
    assert os.listdir(tmp_path) == ["rank0"]


def _fail_on_rank1():
    if dist.get_rank() == 1:
        raise RuntimeError("rank 1 dies")
    dist.barrier()  # never completes: the launcher has to tear this rank down


def test_spawn_propagates_child_failure():
    os.environ["GLOO_SOCKET_TIMEOUT"] = "5"
    with pytest.raises(Exception):
        spawn_parallel_fn(_fail_on_rank1, world_size=2, backend="gloo", master_addr="127.0.0.1", master_port="29622")


def test_single_process_runs_inline():
    seen = []
    spawn_parallel_fn(lambda: seen.append(os.environ["WORLD_SIZE"]), world_size=1, device_type="cpu")
    assert seen == ["1"]


# ---- BASELINE config 1: tiny decoder, next-token training, 10 steps, DDP/FSDP on gloo == single process ----
def _tiny_cfg():
    from khaosz_b200 import AutoRegressiveLMConfig

    return AutoRegressiveLMConfig(vocab_size=1000, dim=128, n_layers=2, norm_eps=1e-5, dim_ffn=384, tie_weight=False,
                                  max_len=128, rope_theta=1e4, n_heads=4, n_kv_heads=2)


def _make_model():
    from khaosz_b200 import AutoRegressiveLM
    from khaosz_b200.models.components.layers import Linear

    torch.manual_seed(3407)
    m = AutoRegressiveLM(_tiny_cfg())
    for mod in m.modules():
        if isinstance(mod, Linear):
            torch.nn.init.normal_(mod.weight, 0.0, 0.02)
    return m


def _run_steps(mode, world, rank, steps=10, accum=1, fused=True, tp_size=None):
    from khaosz_b200.trainer import FusedAdamW, StrategyFactory

    g = torch.Generator().manual_seed(3407)
    # global batch = 2 per data-parallel rank; tensor-parallel ranks all read the same 4 sequences
    data = torch.randint(0, 1000, (steps * accum, 4 if mode == "tp" else 2 * world, 129), generator=g)
    model = _make_model()
    ex = ExecutorFactory.create(mode, grad_accum_steps=accum, **({"tp_size": tp_size} if tp_size else {}))
    if fused:
        opt = FusedAdamW(model.parameters(), lr=1e-4, betas=(0.9, 0.95), weight_decay=0.01)
    else:
        opt = torch.optim.AdamW(model.parameters(), lr=1e-4, betas=(0.9, 0.95), weight_decay=0.01)
    model, opt, _, _ = ex.prepare(model, opt, None, None)
    strat = StrategyFactory.create("seq", model, "cpu", label_smoothing=0.05)
    losses = []
    for i in range(steps * accum):
        if mode == "tp" and tp_size:   # dp x tp: the ranks of one replica share 2 of the 4 sequences
            replica = rank // tp_size
            mine = data[i, 2 * replica:2 * replica + 2]
        else:
            mine = data[i] if mode == "tp" else data[i, 2 * rank:2 * rank + 2]
        with ex.accumulate(model):
            loss = strat({"input_ids": mine[:, :-1], "target_ids": mine[:, 1:]})
            ex.backward(loss / accum)
            if ex.sync_gradients:
                if hasattr(opt, "fused_clip"):
                    opt.fused_clip(1.0)
                else:
                    torch.nn.utils.clip_grad_norm_(model.parameters(), 1.0)
                opt.step()
                opt.zero_grad()
        t = loss.detach().clone()
        if world > 1:
            dist.all_reduce(t)
            t /= world
        losses.append(t.item())
    return losses, {k: v.detach().clone() for k, v in ex.unwrap_model(model).items()}


def _distributed_case(mode, out, tp_size=None):
    losses, sd = _run_steps(mode, dist.get_world_size(), dist.get_rank(), tp_size=tp_size)
    if dist.get_rank() == 0:
        torch.save({"losses": losses, "sd": sd}, out)


def _single_reference():
    """Single process over the *global* batch (4 sequences) == the average of two ranks."""
    from khaosz_b200.trainer import FusedAdamW, StrategyFactory

    g = torch.Generator().manual_seed(3407)
    data = torch.randint(0, 1000, (10, 4, 129), generator=g)
    model = _make_model()
    opt = FusedAdamW(model.parameters(), lr=1e-4, betas=(0.9, 0.95), weight_decay=0.01)
    strat = StrategyFactory.create("seq", model, "cpu", label_smoothing=0.05)
    losses = []
    for i in range(10):
        loss = strat({"input_ids": data[i, :, :-1], "target_ids": data[i, :, 1:]})
        loss.backward()
        opt.fused_clip(1.0)
        opt.step()
        opt.zero_grad()
        losses.append(loss.item())
    return losses, model.state_dict()


@pytest.mark.parametrize("mode,port,world", [("ddp", "29631", 2), ("fsdp", "29632", 2), ("tp", "29633", 2),
                                             ("tp", "29634", 4), ("fsdp_full", "29635", 2),
                                             ("fsdp_zero1", "29636", 2)])  # tp on 4 ranks: 2 KV heads shared by rank pairs
def test_executor_matches_single_process(mode, port, world, tmp_path):
    out = str(tmp_path / "r.pt")
    spawn_parallel_fn(_distributed_case, world_size=world, backend="gloo", master_addr="127.0.0.1", master_port=port,
                      mode=mode, out=out)
    got = torch.load(out)
    ref_losses, ref_sd = _single_reference()
    assert got["losses"] == pytest.approx(ref_losses, rel=2e-4, abs=2e-4)
    assert got["losses"][-1] < got["losses"][0]
    for k, v in ref_sd.items():
        assert torch.allclose(got["sd"][k], v, rtol=1e-3, atol=2e-5), k


def test_tensor_parallel_times_data_parallel_matches_single_process(tmp_path):
    """4 ranks as 2 replicas of a 2-way tensor-parallel model."""
    out = str(tmp_path / "hybrid.pt")
    spawn_parallel_fn(_distributed_case, world_size=4, backend="gloo", master_addr="127.0.0.1", master_port="29638",
                      mode="tp", out=out, tp_size=2)
    got = torch.load(out)
    ref_losses, ref_sd = _single_reference()
    assert got["losses"] == pytest.approx(ref_losses, rel=2e-4, abs=2e-4)
    for k, v in ref_sd.items():
        assert torch.allclose(got["sd"][k], v, rtol=1e-3, atol=2e-5), k


def test_fused_adamw_matches_torch_adamw():
    a, _ = _run_steps("none", 1, 0, steps=4, fused=True)
    b, _ = _run_steps("none", 1, 0, steps=4, fused=False)
    assert a == pytest.approx(b, rel=1e-5, abs=1e-6)


def test_grad_accumulation_equals_big_batch():
    # 2 micro-batches of 2 == one batch of 4 (same data order)
    from khaosz_b200.trainer import FusedAdamW, StrategyFactory

    g = torch.Generator().manual_seed(1)
    data = torch.randint(0, 1000, (2, 2, 129), generator=g)
    m1, m2 = _make_model(), _make_model()
    ex = ExecutorFactory.create("none", grad_accum_steps=2)
    o1 = FusedAdamW(m1.parameters(), lr=1e-3)
    m1, o1, _, _ = ex.prepare(m1, o1, None, None)
    s1 = StrategyFactory.create("seq", m1, "cpu")
    for i in range(2):
        with ex.accumulate(m1):
            ex.backward(s1({"input_ids": data[i, :, :-1], "target_ids": data[i, :, 1:]}) / 2)
            assert ex.sync_gradients == (i == 1)
            o1.step()
            o1.zero_grad()
    o2 = FusedAdamW(m2.parameters(), lr=1e-3)
    s2 = StrategyFactory.create("seq", m2, "cpu")
    big = data.reshape(4, 129)
    s2({"input_ids": big[:, :-1], "target_ids": big[:, 1:]}).backward()
    o2.step()
    for (k, a), b in zip(m1.state_dict().items(), m2.state_dict().values()):
        assert torch.allclose(a, b, rtol=1e-4, atol=1e-6), k


# ---- DPO with a frozen reference copy under the sharded executor (gloo, 2 ranks) ----
def _dpo_fsdp_case(out):
    from khaosz_b200.trainer import FusedAdamW, StrategyFactory

    rank = dist.get_rank()
    model = _make_model()
    ex = ExecutorFactory.create("fsdp", grad_accum_steps=1)
    opt = FusedAdamW(model.parameters(), lr=1e-3)
    model, opt, _, _ = ex.prepare(model, opt, None, None)
    strat = StrategyFactory.create("dpo", model, "cpu", executor=ex, model_fn=_make_model, beta=0.1)
    g = torch.Generator().manual_seed(5 + rank)
    losses = []
    for _ in range(3):
        batch = {"chosen": torch.randint(0, 1000, (2, 48), generator=g), "rejected": torch.randint(0, 1000, (2, 48), generator=g),
                 "chosen_mask": torch.ones(2, 48, dtype=torch.bool), "rejected_mask": torch.ones(2, 48, dtype=torch.bool)}
        with ex.accumulate(model):
            loss = strat(batch)
            ex.backward(loss)
            opt.step()
            opt.zero_grad()
        losses.append(loss.item())
    sd = ex.unwrap_model(model)
    flat = torch.cat([v.reshape(-1).float() for v in sd.values()])
    other = flat.clone()
    dist.broadcast(other, src=0)
    assert torch.equal(flat, other), "ranks diverged after sharded updates"
    if rank == 0:
        torch.save({"losses": losses}, out)


def test_dpo_under_fsdp_keeps_ranks_in_sync(tmp_path):
    out = str(tmp_path / "dpo.pt")
    spawn_parallel_fn(_dpo_fsdp_case, world_size=2, backend="gloo", master_addr="127.0.0.1", master_port="29636", out=out)
    losses = torch.load(out)["losses"]
    assert abs(losses[0] - 0.6931) < 1e-3          # policy == reference at step 0: -log sigmoid(0)
    assert all(l == l and l < 10 for l in losses)


# ---- DPO under tensor parallelism: sequence log-probabilities are gathered over the token slices ----
def _dpo_tp_case(out):
    from khaosz_b200.trainer import FusedAdamW, StrategyFactory

    model = _make_model()
    ex = ExecutorFactory.create("tp", grad_accum_steps=1)
    opt = FusedAdamW(model.parameters(), lr=1e-3)
    model, opt, _, _ = ex.prepare(model, opt, None, None)
    strat = StrategyFactory.create("dpo", model, "cpu", executor=ex, model_fn=_make_model, beta=0.1)
    g = torch.Generator().manual_seed(5)   # every rank reads the same pairs
    losses = []
    for _ in range(3):
        batch = {"chosen": torch.randint(0, 1000, (2, 49), generator=g), "rejected": torch.randint(0, 1000, (2, 49), generator=g),
                 "chosen_mask": torch.ones(2, 49, dtype=torch.bool), "rejected_mask": torch.ones(2, 49, dtype=torch.bool)}
        with ex.accumulate(model):
            loss = ex.micro_step(strat, batch)
            opt.step()
            opt.zero_grad()
        losses.append(loss.item())
    if dist.get_rank() == 0:
        torch.save({"losses": losses, "sd": ex.unwrap_model(model)}, out)
    else:
        ex.unwrap_model(model)


def test_dpo_under_tensor_parallel_matches_single_process(tmp_path):
    from khaosz_b200.trainer import FusedAdamW, StrategyFactory

    out = str(tmp_path / "dpo_tp.pt")
    spawn_parallel_fn(_dpo_tp_case, world_size=2, backend="gloo", master_addr="127.0.0.1", master_port="29637", out=out)
    got = torch.load(out)
    model = _make_model()
    opt = FusedAdamW(model.parameters(), lr=1e-3)
    ex = ExecutorFactory.create("none")
    model, opt, _, _ = ex.prepare(model, opt, None, None)
    strat = StrategyFactory.create("dpo", model, "cpu", executor=ex, model_fn=_make_model, beta=0.1)
    g = torch.Generator().manual_seed(5)
    ref = []
    for _ in range(3):
        batch = {"chosen": torch.randint(0, 1000, (2, 49), generator=g), "rejected": torch.randint(0, 1000, (2, 49), generator=g),
                 "chosen_mask": torch.ones(2, 49, dtype=torch.bool), "rejected_mask": torch.ones(2, 49, dtype=torch.bool)}
        loss = strat(batch)
        loss.backward()
        opt.step()
        opt.zero_grad()
        ref.append(loss.item())
    assert got["losses"] == pytest.approx(ref, rel=1e-3, abs=1e-4)
    # Adam divides by tiny second moments here (policy == reference at the start), so rounding
    # differences of the gradients are amplified: three steps of lr 1e-3 move a weight by up to 3e-3
    for k, v in model.state_dict().items():
        assert torch.allclose(got["sd"][k], v, rtol=1e-3, atol=3e-4), k


# ---- optimizer state of a tensor-parallel run survives a checkpoint written by rank 0 ----
def _tp_opt_state_case(out, mode="tp"):
    from khaosz_b200.trainer import FusedAdamW, StrategyFactory

    def fresh():
        model = _make_model()
        ex = ExecutorFactory.create(mode, grad_accum_steps=1)
        opt = FusedAdamW(model.parameters(), lr=1e-3)
        model, opt, _, _ = ex.prepare(model, opt, None, None)
        return model, ex, opt

    model, ex, opt = fresh()
    strat = StrategyFactory.create("seq", model, "cpu")
    data = torch.randint(0, 1000, (2, 4, 65), generator=torch.Generator().manual_seed(1))
    for i in range(2):
        mine = data[i] if mode == "tp" else data[i, 2 * dist.get_rank():2 * dist.get_rank() + 2]
        with ex.accumulate(model):
            ex.micro_step(strat, {"input_ids": mine[:, :-1], "target_ids": mine[:, 1:]})
            opt.step()
            opt.zero_grad()
    state = opt.state_dict()                      # collective: the dense model's optimizer.pt layout
    dense_shapes = [tuple(p.shape) for p in _make_model().parameters()]
    assert [tuple(state["state"][i]["exp_avg"].shape) for i in range(len(dense_shapes))] == dense_shapes
    if dist.get_rank() == 0:
        torch.save(state, out)                    # only rank 0 writes, as the checkpoint callback does
    dist.barrier()
    state = torch.load(out, weights_only=False)
    model2, ex2, opt2 = fresh()
    opt2.load_state_dict(state)
    a, b = opt.optimizer.state_dict(), opt2.optimizer.state_dict()
    for i in a["state"]:
        assert torch.equal(a["state"][i]["exp_avg"], b["state"][i]["exp_avg"]), i
        assert torch.equal(a["state"][i]["exp_avg_sq"], b["state"][i]["exp_avg_sq"]), i
    # the two ranks really hold different moments for the sharded weights
    mine = sum(st["exp_avg"].double().abs().sum() for st in a["state"].values()).float()
    both = [torch.zeros(()) for _ in range(2)]
    dist.all_gather(both, mine)
    assert not torch.equal(both[0], both[1])


@pytest.mark.parametrize("mode,port", [("tp", "29639"), ("fsdp_full", "29640")])
def test_sharded_optimizer_state_roundtrip(mode, port, tmp_path):
    spawn_parallel_fn(_tp_opt_state_case, world_size=2, backend="gloo", master_addr="127.0.0.1", master_port=port,
                      out=str(tmp_path / "opt.pt"), mode=mode)


# ---- tensor parallelism with QK-RMSNorm and the sigmoid output gate ----
def _tp_variant_case(out, moe=False, mla=False):
    from khaosz_b200 import AutoRegressiveLM, AutoRegressiveLMConfig
    from khaosz_b200.parallel.tp_model import tensorize
    from khaosz_b200.trainer import StrategyFactory

    ffn = dict(ffn_type="moe", n_routed_experts=4, n_shared_experts=1, n_activated_experts=2) if moe else {}
    cfg = AutoRegressiveLMConfig(vocab_size=200, dim=64, n_layers=2, norm_eps=1e-5, dim_ffn=128, tie_weight=False,
                                 max_len=64, rope_theta=1e4, n_heads=4, n_kv_heads=2, use_qk_norm=True,
                                 use_gated_attention=True, **ffn,
                                 **(dict(attn_type="mla", kv_lora_rank=16, qk_nope_head_dim=8, qk_rope_head_dim=8) if mla else {}))
    torch.manual_seed(21)
    dense = AutoRegressiveLM(cfg)
    with torch.no_grad():   # norm weights away from one, so that their gradients are not trivially alike
        for name, p in dense.named_parameters():
            if "norm" in name:
                p.add_(0.1 * torch.randn_like(p))
    data = torch.randint(0, 200, (4, 33), generator=torch.Generator().manual_seed(2))
    batch = {"input_ids": data[:, :-1], "target_ids": data[:, 1:]}
    ref_loss = StrategyFactory.create("seq", dense, "cpu")(batch)
    ref_loss.backward()
    ref = {n: p.grad.clone() for n, p in dense.named_parameters()}
    dense.zero_grad()

    tp = tensorize(dense)
    loss = StrategyFactory.create("seq", tp, "cpu")(batch)
    (loss / dist.get_world_size()).backward()
    tp.reduce_replicated_grads()
    got = tp.full_state_dict(grads=True)
    total = loss.detach().clone()
    dist.all_reduce(total)
    weights = tp.full_state_dict()
    back = tp.scatter_named(weights)             # the inverse: every local parameter from the dense-named tensors
    for prm in tp.parameters():
        assert torch.equal(back[id(prm)], prm), "scatter_named does not invert gather_named"
    if dist.get_rank() == 0:
        torch.save({"loss": total.item() / dist.get_world_size(), "ref_loss": ref_loss.item(), "got": got, "ref": ref,
                    "names": sorted(weights), "dense_names": sorted(n for n, _ in dense.named_parameters())}, out)
    dist.barrier()


@pytest.mark.parametrize("world,port,moe,mla", [
    (2, "29644", False, False), (4, "29645", False, False),   # 4 ranks: KV heads shared by rank pairs
    (2, "29648", True, False),                                # mixture of experts: replicated experts on token slices
    (2, "29649", False, True)])                               # multi-head latent attention
def test_tensor_parallel_qk_norm_and_gate_match_the_dense_model(world, port, moe, mla, tmp_path):
    out = str(tmp_path / "variant.pt")
    spawn_parallel_fn(_tp_variant_case, world_size=world, backend="gloo", master_addr="127.0.0.1", master_port=port, out=out,
                      moe=moe, mla=mla)
    r = torch.load(out)
    assert r["loss"] == pytest.approx(r["ref_loss"], rel=1e-4)
    assert r["names"] == r["dense_names"]
    for k, v in r["ref"].items():
        assert torch.allclose(r["got"][k], v, rtol=1e-3, atol=1e-6), k


def _fs_variant_case(out, variant="gqa"):
    from khaosz_b200 import AutoRegressiveLM, AutoRegressiveLMConfig
    from khaosz_b200.parallel.fsdp_model import full_shard
    from khaosz_b200.trainer import StrategyFactory

    extra = {}
    if variant == "mla_moe":
        extra = dict(attn_type="mla", kv_lora_rank=16, qk_nope_head_dim=8, qk_rope_head_dim=8, ffn_type="moe",
                     n_routed_experts=4, n_shared_experts=1, n_activated_experts=2)
    cfg = AutoRegressiveLMConfig(vocab_size=200, dim=64, n_layers=2, norm_eps=1e-5, dim_ffn=128, tie_weight=False,
                                 max_len=64, rope_theta=1e4, n_heads=4, n_kv_heads=2, use_qk_norm=True,
                                 use_gated_attention=True, **extra)
    torch.manual_seed(21)
    dense = AutoRegressiveLM(cfg)
    data = torch.randint(0, 200, (4, 33), generator=torch.Generator().manual_seed(2))
    ref_loss = StrategyFactory.create("seq", dense, "cpu")({"input_ids": data[:, :-1], "target_ids": data[:, 1:]})
    ref_loss.backward()
    ref = {n: p.grad.clone() for n, p in dense.named_parameters()}
    dense.zero_grad()

    fs = full_shard(dense)
    ws, r = dist.get_world_size(), dist.get_rank()
    mine = data[2 * r:2 * r + 2]                     # data parallel: every rank its own two sequences
    loss = StrategyFactory.create("seq", fs, "cpu")({"input_ids": mine[:, :-1], "target_ids": mine[:, 1:]})
    (loss / ws).backward()
    fs.reduce_replicated_grads()
    got = fs.gather_named(lambda p: p.grad.detach())
    back = fs.scatter_named(fs.full_state_dict())
    for prm in fs.parameters():
        assert torch.equal(back[id(prm)], prm), "scatter_named does not invert gather_named"
    if r == 0:
        torch.save({"got": got, "ref": ref}, out)
    dist.barrier()   # leave together: a rank that tears gloo down while its peer still writes aborts the peer


@pytest.mark.parametrize("variant,port", [("gqa", "29647"), ("mla_moe", "29681")])
def test_full_shard_qk_norm_and_gate_match_the_dense_model(variant, port, tmp_path):
    out = str(tmp_path / "fs_variant.pt")
    spawn_parallel_fn(_fs_variant_case, world_size=2, backend="gloo", master_addr="127.0.0.1", master_port=port, out=out,
                      variant=variant)
    r = torch.load(out)
    assert sorted(r["got"]) == sorted(r["ref"])
    for k, v in r["ref"].items():
        assert torch.allclose(r["got"][k], v, rtol=1e-3, atol=1e-6), k


def test_sliced_models_refuse_lora_adapters_instead_of_dropping_them():
    from khaosz_b200 import AutoRegressiveLM
    from khaosz_b200.models.components.lora import inject_lora, merge_lora
    from khaosz_b200.parallel.tp_model import reject_adapters

    model = AutoRegressiveLM(_tiny_cfg())
    reject_adapters(model, "tensor parallelism")          # nothing wrapped: fine
    inject_lora(model, r=4, alpha=8)
    with pytest.raises(NotImplementedError, match="LoRA adapters"):
        reject_adapters(model, "tensor parallelism")
    merge_lora(model)                                      # merged adapters are plain weights again
    reject_adapters(model, "tensor parallelism")


# ---- the frozen reference copy of DPO / GRPO is cut like the policy ----
def _sharded_ref_case(mode):
    from khaosz_b200.parallel.fsdp_model import FullShardLM
    from khaosz_b200.parallel.tp_model import TensorParallelLM
    from khaosz_b200.trainer import FusedAdamW, StrategyFactory

    model = _make_model()
    ex = ExecutorFactory.create(mode, grad_accum_steps=1)
    opt = FusedAdamW(model.parameters(), lr=1e-3)
    model, opt, _, _ = ex.prepare(model, opt, None, None)
    strat = StrategyFactory.create("dpo", model, "cpu", executor=ex, model_fn=_make_model, beta=0.1)
    seed = 5 if mode == "tp" else 5 + dist.get_rank()       # data parallel: every rank its own pairs
    g = torch.Generator().manual_seed(seed)
    batch = {"chosen": torch.randint(0, 1000, (2, 33), generator=g), "rejected": torch.randint(0, 1000, (2, 33), generator=g),
             "chosen_mask": torch.ones(2, 33, dtype=torch.bool), "rejected_mask": torch.ones(2, 33, dtype=torch.bool)}
    with ex.accumulate(model):
        loss = ex.micro_step(strat, batch)
        opt.step()
    ref = strat.ref_model
    assert isinstance(ref, TensorParallelLM if mode == "tp" else FullShardLM)
    assert not any(p.requires_grad for p in ref.parameters())
    dense = sum(p.numel() for p in _make_model().layers.parameters())
    held = sum(p.numel() for p in ref.layers.parameters())
    assert held < 0.6 * dense                                # two ranks: about half of every block
    # policy == reference before the first update: the DPO loss is log 2
    assert loss.item() == pytest.approx(0.6931, abs=2e-3)
    # GRPO refreshes its old-policy copy in place: after a refresh it holds the updated weights, piece by piece
    grpo = StrategyFactory.create("grpo", model, "cpu", executor=ex, model_fn=_make_model, group_size=4, sync_interval=1)
    before = [p.detach().clone() for p in grpo.ref_model.parameters()]
    with torch.no_grad():
        for prm in model.parameters():                                       # the policy moves on
            prm.add_(0.01)
    grpo.sync_ref_model()
    after = list(grpo.ref_model.parameters())
    assert all(not torch.equal(a, b) for a, b in zip(after, before))
    for mine, pol in zip(grpo.ref_model.layers.parameters(), model.layers.parameters()):
        assert torch.equal(mine, pol)


@pytest.mark.parametrize("mode,port", [("tp", "29682"), ("fsdp_full", "29683")])
def test_frozen_reference_model_is_sharded_like_the_policy(mode, port):
    spawn_parallel_fn(_sharded_ref_case, world_size=2, backend="gloo", master_addr="127.0.0.1", master_port=port, mode=mode)


# ---- SFT under tensor parallelism: the masked positions fall unevenly on the ranks' token slices ----
def _sft_tp_case():
    from khaosz_b200.parallel.tp_model import tensorize
    from khaosz_b200.trainer import StrategyFactory

    dense = _make_model()
    data = torch.randint(0, 1000, (4, 65), generator=torch.Generator().manual_seed(9))
    mask = torch.ones(4, 64, dtype=torch.bool)
    mask[:2] = False                      # the first rank's token slice is all context ...
    mask[0, 60:] = True                   # ... except four positions
    batch = {"input_ids": data[:, :-1], "target_ids": data[:, 1:], "loss_mask": mask}
    ref = StrategyFactory.create("sft", dense, "cpu")(batch)
    ref.backward()
    want = dense.layers[0].mlp.down.weight.grad.clone()
    dense.zero_grad()
    tp = tensorize(dense)
    loss = StrategyFactory.create("sft", tp, "cpu")(batch)
    (loss / dist.get_world_size()).backward()
    tp.reduce_replicated_grads()
    got = tp.full_state_dict(grads=True)["layers.0.mlp.down.weight"]
    total = loss.detach().clone()
    dist.all_reduce(total)
    assert total.item() / dist.get_world_size() == pytest.approx(ref.item(), rel=1e-5)
    assert torch.allclose(got, want, rtol=1e-3, atol=1e-7)
    dist.barrier()


def test_sft_under_tensor_parallel_weights_uneven_masks_exactly():
    spawn_parallel_fn(_sft_tp_case, world_size=2, backend="gloo", master_addr="127.0.0.1", master_port="29684")


# ---- GRPO under tensor parallelism ----
def _grpo_batch():
    g = torch.Generator().manual_seed(3)
    return {"prompts": torch.randint(0, 1000, (2, 6), generator=g), "responses": torch.randint(0, 1000, (2, 4, 11), generator=g),
            "masks": torch.rand(2, 4, 11, generator=g) > 0.2, "rewards": torch.rand(2, 4, generator=g)}


def _grpo_tp_case(out, sync_interval=100):
    from khaosz_b200.trainer import FusedAdamW, StrategyFactory

    model = _make_model()
    ex = ExecutorFactory.create("tp", grad_accum_steps=1)
    opt = FusedAdamW(model.parameters(), lr=1e-3)
    model, opt, _, _ = ex.prepare(model, opt, None, None)
    strat = StrategyFactory.create("grpo", model, "cpu", executor=ex, model_fn=_make_model, group_size=4, kl_coef=0.1,
                                   sync_interval=sync_interval)
    losses = []
    for _ in range(3):
        with ex.accumulate(model):
            losses.append(ex.micro_step(strat, _grpo_batch()).item())
            opt.step()
            opt.zero_grad()
    sd = ex.unwrap_model(model)
    if dist.get_rank() == 0:
        torch.save({"losses": losses, "sd": sd}, out)


@pytest.mark.parametrize("sync_interval,port", [(100, "29685"), (2, "29688")])   # 2: the old-policy copy is refreshed mid-run
def test_grpo_under_tensor_parallel_matches_single_process(sync_interval, port, tmp_path):
    from khaosz_b200.trainer import FusedAdamW, StrategyFactory

    out = str(tmp_path / "grpo_tp.pt")
    spawn_parallel_fn(_grpo_tp_case, world_size=2, backend="gloo", master_addr="127.0.0.1", master_port=port, out=out,
                      sync_interval=sync_interval)
    got = torch.load(out)
    model = _make_model()
    opt = FusedAdamW(model.parameters(), lr=1e-3)
    ex = ExecutorFactory.create("none")
    model, opt, _, _ = ex.prepare(model, opt, None, None)
    strat = StrategyFactory.create("grpo", model, "cpu", executor=ex, model_fn=_make_model, group_size=4, kl_coef=0.1,
                                   sync_interval=sync_interval)
    ref = []
    for _ in range(3):
        loss = strat(_grpo_batch())
        loss.backward()
        opt.step()
        opt.zero_grad()
        ref.append(loss.item())
    assert got["losses"] == pytest.approx(ref, rel=1e-3, abs=1e-5)
    assert abs(ref[-1]) > 1e-6 or sync_interval == 2     # the policy has moved away from the reference copy
    for k, v in model.state_dict().items():
        assert torch.allclose(got["sd"][k], v, rtol=1e-3, atol=3e-4), k


# ---- the optimizer state of a single-process run loads into tensor-parallel / fully sharded runs ----
def _dense_state_into_sharded_case(path, mode):
    from khaosz_b200.trainer import FusedAdamW

    dense = torch.load(path, weights_only=False)
    model = _make_model()
    ex = ExecutorFactory.create(mode, grad_accum_steps=1)
    opt = FusedAdamW(model.parameters(), lr=1e-3)
    model, opt, _, _ = ex.prepare(model, opt, None, None)
    opt.load_state_dict(dense)                           # every rank takes its slices
    back = opt.state_dict()                              # collective: reassembled to the dense layout
    assert len(back["state"]) == len(dense["state"])
    for i, st in dense["state"].items():
        assert torch.equal(back["state"][i]["exp_avg"], st["exp_avg"]), i
        assert torch.equal(back["state"][i]["exp_avg_sq"], st["exp_avg_sq"]), i
        assert int(back["state"][i]["step"]) == int(st["step"])
    assert back["param_groups"][0]["lr"] == dense["param_groups"][0]["lr"]
    dist.barrier()


@pytest.mark.parametrize("mode,port", [("tp", "29686"), ("fsdp_full", "29687"), ("fsdp", "29688")])
def test_dense_optimizer_state_loads_into_sharded_runs(mode, port, tmp_path):
    from khaosz_b200.trainer import FusedAdamW, StrategyFactory

    model = _make_model()
    opt = FusedAdamW(model.parameters(), lr=1e-3)
    strat = StrategyFactory.create("seq", model, "cpu")
    data = torch.randint(0, 1000, (2, 4, 65), generator=torch.Generator().manual_seed(1))
    for i in range(2):
        strat({"input_ids": data[i, :, :-1], "target_ids": data[i, :, 1:]}).backward()
        opt.step()
        opt.zero_grad()
    path = str(tmp_path / "dense_opt.pt")
    torch.save(opt.state_dict(), path)
    spawn_parallel_fn(_dense_state_into_sharded_case, world_size=2, backend="gloo", master_addr="127.0.0.1",
                      master_port=port, path=path, mode=mode)


def test_bucketed_ownership_layout_matches_the_kernel_mapping():
    """Rank r owns sub-slice r of every gradient bucket; the optimizer-state layout that the checkpoint code
    uses (``owned_ranges``) must be the mapping the update kernel computes (local element -> global element)."""
    from types import SimpleNamespace

    from khaosz_b200.parallel.comm import GradReducer

    for ws, numel, bucket_n in [(2, 16 * 37, 16 * 10), (8, 64 * 50, 64 * 7), (4, 32 * 9, 32 * 9), (8, 64 * 3, 64 * 100)]:
        bucket_n = min(bucket_n, numel)
        covered = torch.zeros(numel, dtype=torch.int32)
        for rank in range(ws):
            r = GradReducer.__new__(GradReducer)
            r.flat = SimpleNamespace(numel=numel)
            r.ws, r.rank, r.bucket_n = ws, rank, bucket_n
            r.n_buckets = -(-numel // bucket_n)
            ranges = r.owned_ranges()
            assert sum(n for _, _, n in ranges) == numel // ws
            per = bucket_n // ws
            for g, l, n in ranges:
                covered[g:g + n] += 1
                for i in (l, l + n - 8):          # first and last 8-element chunk of the piece, as the kernel maps them
                    b = i // per
                    len_b = min(bucket_n, numel - b * bucket_n)
                    assert b * bucket_n + rank * (len_b // ws) + (i - b * per) == g + (i - l)
        assert bool((covered == 1).all())             # the ranks' pieces tile the vector exactly once
