"""Bandwidth-bound kernels vs plain fp32 PyTorch references."""
import pytest
import torch
import torch.nn.functional as F

from khaosz_b200 import ops
from khaosz_b200.ops import functional as KF

pytestmark = pytest.mark.gpu


def _close(got, ref, rtol=2e-2, atol=2e-2):
    err = (got.float() - ref.float()).abs().max().item()
    lim = rtol * ref.float().abs().max().item() + atol
    assert err <= lim, f"max err {err} > {lim}"


@pytest.mark.parametrize("rows,dim", [(64, 2048), (1000, 512), (7, 128), (33, 4096)])
def test_rmsnorm_fwd_bwd(rows, dim):
    x = torch.randn(rows, dim, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    w = (1 + 0.1 * torch.randn(dim, device="cuda")).to(torch.bfloat16).requires_grad_()
    y = ops.rms_norm(x, w, 1e-5)
    g = torch.randn_like(y)
    y.backward(g)
    xf, wf = x.detach().float().requires_grad_(), w.detach().float().requires_grad_()
    yf = F.rms_norm(xf, (dim,), wf, 1e-5)
    yf.backward(g.float())
    _close(y, yf)
    _close(x.grad, xf.grad)
    _close(w.grad, wf.grad, rtol=3e-2, atol=0.3)


def test_add_rmsnorm_fwd_bwd():
    rows, dim = 300, 2048
    x = torch.randn(rows, dim, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    r = torch.randn(rows, dim, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    w = torch.ones(dim, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    y, s = ops.add_rms_norm(x, r, w, 1e-5)
    g1, g2 = torch.randn_like(y), torch.randn_like(s)
    (y * g1 + s * g2).sum().backward()
    xf, rf, wf = (t.detach().float().requires_grad_() for t in (x, r, w))
    sf = xf + rf
    yf = F.rms_norm(sf, (dim,), wf, 1e-5)
    (yf * g1.float() + sf * g2.float()).sum().backward()
    _close(y, yf)
    _close(s, sf)
    _close(x.grad, xf.grad, atol=5e-2)
    _close(r.grad, rf.grad, atol=5e-2)


def test_rope_matches_complex_rotation():
    B, S, H, D = 2, 64, 6, 128
    x = torch.randn(B, S, H, D, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    cs = ops.rope_table(D, 256, 10000.0, device="cuda")
    y = ops.rope(x, cs)
    freqs = torch.view_as_complex(cs[:S].contiguous())  # cos + i sin
    xc = torch.view_as_complex(x.detach().float().reshape(B, S, H, D // 2, 2))
    ref = torch.view_as_real(xc * freqs[None, :, None, :]).reshape(B, S, H, D)
    _close(y, ref)
    g = torch.randn_like(y)
    y.backward(g)
    gc = torch.view_as_complex(g.float().reshape(B, S, H, D // 2, 2))
    gref = torch.view_as_real(gc * freqs.conj()[None, :, None, :]).reshape(B, S, H, D)
    _close(x.grad, gref)
    # explicit positions and partial-head rotation
    pos = torch.randint(0, 256, (B, S), device="cuda")
    y2 = ops.rope(x.detach(), cs, pos, n_heads=4)
    ref2 = KF._rope_torch(x.detach().float()[:, :, :4], cs, pos)
    _close(y2[:, :, :4], ref2)
    assert torch.equal(y2[:, :, 4:], x.detach()[:, :, 4:])


def test_swiglu_fwd_bwd():
    gu = torch.randn(257, 2 * 1408, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    h = ops.swiglu(gu)
    g = torch.randn_like(h)
    h.backward(g)
    guf = gu.detach().float().requires_grad_()
    hf = guf[:, 1408:] * F.silu(guf[:, :1408])
    hf.backward(g.float())
    _close(h, hf)
    _close(gu.grad, guf.grad)


@pytest.mark.parametrize("V,smoothing", [(32000, 0.0), (32000, 0.1), (1000, 0.05), (1003, 0.0)])
def test_cross_entropy_fwd_bwd(V, smoothing):
    rows = 96
    ld = (V + 7) // 8 * 8
    buf = torch.randn(rows, ld, device="cuda", dtype=torch.bfloat16) * 3
    logits = buf[:, :V].detach().requires_grad_()
    t = torch.randint(0, V, (rows,), device="cuda")
    t[::7] = -100
    ref_in = logits.detach().float().requires_grad_()
    ref = F.cross_entropy(ref_in, t, label_smoothing=smoothing, ignore_index=-100)
    ref.backward()
    loss = ops.cross_entropy(logits, t, smoothing, -100)
    loss.backward()
    assert abs(loss.item() - ref.item()) <= 2e-3 * abs(ref.item()) + 1e-3
    _close(logits.grad, ref_in.grad, rtol=2e-2, atol=1e-5)


def test_token_logprobs_fwd_bwd():
    B, S, V = 3, 17, 4096
    logits = (torch.randn(B, S, V, device="cuda", dtype=torch.bfloat16) * 2).requires_grad_()
    t = torch.randint(0, V, (B, S), device="cuda")
    ref_in = logits.detach().float().requires_grad_()
    ref = torch.log_softmax(ref_in, -1).gather(-1, t[..., None]).squeeze(-1)
    w = torch.randn(B, S, device="cuda")
    (ref * w).sum().backward()
    lp = ops.token_logprobs(logits, t)
    (lp * w).sum().backward()
    _close(lp, ref, rtol=1e-3, atol=2e-3)
    _close(logits.grad, ref_in.grad, rtol=2e-2, atol=1e-4)


def test_embedding_fwd_bwd():
    V, D = 1000, 256
    table = torch.randn(V, D, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    ids = torch.randint(0, V, (4, 64), device="cuda")
    out = ops.embedding(ids, table)
    assert torch.equal(out, table.detach()[ids])
    g = torch.randn_like(out)
    out.backward(g)
    tf = table.detach().float().requires_grad_()
    F.embedding(ids, tf).backward(g.float())
    _close(table.grad, tf.grad)


def test_fp8_forward_linear_matches_bf16_within_fp8_error():
    """The fp8 switch changes only the forward GEMM: outputs agree with bf16 to e4m3 precision and
    the gradients (bf16 GEMMs on the same saved operands) are identical in form."""
    from khaosz_b200.ops import set_fp8_linear

    torch.manual_seed(0)
    x = (torch.randn(512, 1024, device="cuda") * 0.5).to(torch.bfloat16).requires_grad_()
    w = (torch.randn(768, 1024, device="cuda") * 0.05).to(torch.bfloat16).requires_grad_()
    ref = ops.linear(x, w)
    gref = torch.autograd.grad(ref.float().pow(2).sum(), (x, w))
    set_fp8_linear(True)
    try:
        out = ops.linear(x, w)
        g = torch.autograd.grad(out.float().pow(2).sum(), (x, w))
    finally:
        set_fp8_linear(False)
    full = x.float() @ w.float().t()
    rel = (out.float() - full).norm() / full.norm()
    assert rel < 0.06, rel            # e4m3 has 3 mantissa bits
    assert (ref.float() - full).norm() / full.norm() < 0.01
    for a, b in zip(g, gref):
        assert (a.float() - b.float()).norm() / b.float().norm() < 0.08


def test_cuda_graph_micro_step_matches_plain_launches():
    """Executor option cuda_graph: the captured forward+backward gives the same losses and weights."""
    from khaosz_b200 import AutoRegressiveLM, AutoRegressiveLMConfig
    from khaosz_b200.parallel import ExecutorFactory
    from khaosz_b200.trainer import FusedAdamW, StrategyFactory

    cfg = AutoRegressiveLMConfig(vocab_size=2048, dim=256, n_layers=2, norm_eps=1e-5, dim_ffn=768, tie_weight=True,
                                 max_len=128, rope_theta=1e4, n_heads=2, n_kv_heads=1)
    data = torch.randint(0, 2048, (8, 2, 129), generator=torch.Generator().manual_seed(1)).cuda()

    def run(graph):
        torch.manual_seed(0)
        model = AutoRegressiveLM(cfg).to(device="cuda", dtype=torch.bfloat16)
        ex = ExecutorFactory.create("none", grad_accum_steps=2, cuda_graph=graph)
        opt = FusedAdamW(model.parameters(), lr=1e-3)
        model, opt, _, _ = ex.prepare(model, opt, None, None)
        strat = StrategyFactory.create("seq", model, "cuda")
        losses = []
        for i in range(8):
            with ex.accumulate(model):
                loss = ex.micro_step(strat, {"input_ids": data[i, :, :-1].contiguous(), "target_ids": data[i, :, 1:].contiguous()})
                if ex.sync_gradients:
                    opt.step()
                    opt.zero_grad()
            losses.append(loss.item())
        if graph:
            assert not ex._graphed.disabled and any("graph" in e for e in ex._graphed.entries.values())
        return losses, torch.cat([p.detach().float().reshape(-1) for p in model.parameters()])

    l0, w0 = run(False)
    l1, w1 = run(True)
    assert l0 == pytest.approx(l1, rel=1e-3, abs=1e-3)
    assert (w0 - w1).abs().max().item() < 1e-2


def test_rms_norm_fork_fuses_the_residual_gradient():
    torch.manual_seed(3)
    x = torch.randn(300, 512, device="cuda").to(torch.bfloat16).requires_grad_()
    w = (1 + 0.1 * torch.randn(512, device="cuda")).to(torch.bfloat16).requires_grad_()
    a = torch.randn(300, 512, device="cuda").to(torch.bfloat16)
    b = torch.randn(300, 512, device="cuda").to(torch.bfloat16)
    y, xr = ops.rms_norm_fork(x, w, 1e-5)
    gx, gw = torch.autograd.grad((y.float() * a.float()).sum() + (xr.float() * b.float()).sum(), (x, w))
    xf, wf = x.detach().float().requires_grad_(), w.detach().float().requires_grad_()
    ref = F.rms_norm(xf, (512,), wf, 1e-5)
    rx, rw = torch.autograd.grad((ref * a.float()).sum() + (xf * b.float()).sum(), (xf, wf))
    assert torch.equal(xr, x)
    assert (gx.float() - rx).abs().max().item() < 3e-2 * rx.abs().max().item() + 2e-2
    assert (gw.float() - rw).abs().max().item() < 3e-2 * rw.abs().max().item() + 0.5


def test_throughput_callback_times_steps_on_the_device():
    """The trainer's throughput callback brackets optimizer steps with CUDA events and reads an interval
    only once both of its events have completed."""
    from types import SimpleNamespace

    from khaosz_b200.trainer import CallbackFactory

    cb = CallbackFactory.create("throughput")
    ctx = SimpleNamespace(kwargs={"batch_tokens": 1024}, world_size=1, dataloader=None)
    x = torch.randn(2048, 2048, device="cuda")
    for _ in range(4):
        cb.on_batch_end(ctx)
        (x @ x).sum()
        cb.on_optimizer_step(ctx)
        torch.cuda.synchronize()
    assert cb._use_cuda and len(cb._marks) <= 2
    assert 0 < ctx.kwargs["step_ms"] < 1000 and ctx.kwargs["tokens_per_s"] > 0


def test_adamw_kernel_tracks_fp32_adamw_over_30_steps():
    """The library is compiled with fast-math; the optimizer kernel's divisions, square roots and powers
    must still follow an AdamW computed in double precision over many steps.  The moments do not depend
    on the parameters, so they are compared at the end (fp32 accuracy).  bf16 parameters are compared
    step by step, each step starting from the kernel's own previous parameters: two trajectories that
    round one tie differently stay apart for good (a bf16 weight whose update is half an ulp stalls on
    one side of a binade boundary and keeps moving on the other), which says nothing about the kernel."""
    from khaosz_b200.ops._lib import check, lib, ptr, stream

    n, steps = 1 << 20, 30
    lr, b1, b2, eps, wd = 3e-4, 0.9, 0.95, 1e-8, 0.01
    g = torch.Generator(device="cuda").manual_seed(11)
    p = (torch.randn(n, device="cuda", generator=g) * 0.02).to(torch.bfloat16)
    start = p.clone()
    m = torch.zeros(n, device="cuda")
    v = torch.zeros(n, device="cuda")
    m_ref, v_ref = m.double(), v.double()
    lr_step = torch.zeros(2, device="cuda")
    flips = 0
    for t in range(1, steps + 1):
        grad = (torch.randn(n, device="cuda", generator=g) * (1e-3 if t % 3 else 1e-1)).to(torch.bfloat16)
        before = p.clone()
        lr_step.copy_(torch.tensor([lr, float(t)]))
        check(lib().kb_adamw_bf16(ptr(p), ptr(grad), ptr(m), ptr(v), n, ptr(lr_step), b1, b2, eps, wd, 1.0, None, 0.0,
                                  stream()), "adamw")
        gd = grad.double()
        m_ref = b1 * m_ref + (1 - b1) * gd
        v_ref = b2 * v_ref + (1 - b2) * gd * gd
        bc1, bc2 = 1 - b1 ** t, 1 - b2 ** t
        exact = before.double() * (1 - lr * wd) - (lr / bc1) * m_ref / (v_ref.sqrt() / bc2 ** 0.5 + eps)
        want = exact.to(torch.bfloat16).float()
        # the kernel's fp32 result before rounding is within a few fp32 roundings of `exact`, measured at the
        # size of the terms (old parameter, update): where the two cancel, the result is tiny and its own bf16
        # step is smaller than that error, which then shows as several steps of a number near zero
        fp32_error = 2e-6 * (before.double().abs() + lr)
        cancelled = (p.double() - exact).abs() <= fp32_error
        # everywhere else the stored value is the correctly rounded one or, at a tie, its neighbour
        scale = torch.maximum(want.abs(), p.float().abs()).clamp_min(1e-30)
        ulp = torch.exp2(torch.floor(torch.log2(scale)) - 7)
        off = (p.float() - want).abs() / ulp
        bad = (off > 1.0) & ~cancelled
        if bad.any():
            i = int(torch.nonzero(bad)[0])
            raise AssertionError(f"step {t}: {int(bad.sum())} elements off by more than one bf16 step, e.g. before "
                                 f"{before[i].item()!r} exact {exact[i].item()!r} kernel {p[i].item()!r} grad {grad[i].item()!r}")
        differs = (off > 0) & ~cancelled
        flips += int(differs.sum().item())
        if differs.any():       # a neighbour is only acceptable when the exact value sat at the tie
            mid = (p.float().double() + want.double()) / 2
            assert ((exact - mid).abs()[differs] <= fp32_error[differs]).all(), t
    torch.cuda.synchronize()
    assert (m.double() - m_ref).abs().max().item() <= 1e-5 * m_ref.abs().max().item()
    assert (v.double() - v_ref).abs().max().item() <= 1e-5 * v_ref.abs().max().item()
    assert flips < 1e-4 * n * steps, flips                 # ties are rare
    assert (p.float() - start.float()).abs().max().item() > 10 * lr       # the parameters did move
