"""tcgen05 flash attention (forward / backward) vs fp32 softmax attention."""
import math

import pytest
import torch

from khaosz_b200 import ops
from khaosz_b200.ops import attention as A

pytestmark = pytest.mark.gpu


def _mk(B, S, H, Hkv, D=128, seed=0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    qkv = torch.randn(B, S, H + 2 * Hkv, D, device="cuda", generator=g).to(torch.bfloat16)
    return qkv, qkv[:, :, :H], qkv[:, :, H:H + Hkv], qkv[:, :, H + Hkv:]


@pytest.mark.parametrize("B,S,H,Hkv", [(1, 128, 2, 1), (2, 256, 4, 2), (1, 512, 4, 1), (2, 384, 3, 3), (1, 200, 2, 2),
                                       (1, 1024, 8, 2)])
@pytest.mark.parametrize("causal", [True, False])
def test_flash_forward(B, S, H, Hkv, causal):
    _, q, k, v = _mk(B, S, H, Hkv)
    o, lse = A._flash_fwd(q, k, v, causal, 1.0 / math.sqrt(128))
    torch.cuda.synchronize()
    ops.raise_on_device_error()
    ref = ops.sdpa_reference(q, k, v, causal)
    err = (o.float() - ref.float()).abs().max().item()
    assert err < 2e-2, f"max err {err}"
    # log-sum-exp against the dense computation
    qf = q.float().permute(0, 2, 1, 3)
    kf = k.float().permute(0, 2, 1, 3).repeat_interleave(H // Hkv, 1)
    s = qf @ kf.transpose(-1, -2) / math.sqrt(128)
    if causal:
        s = s.masked_fill(~torch.ones(S, S, dtype=torch.bool, device="cuda").tril(), float("-inf"))
    assert (lse - torch.logsumexp(s, -1)).abs().max().item() < 2e-2


def test_flash_forward_throughput_report():
    B, S, H, Hkv = 4, 2048, 16, 4
    _, q, k, v = _mk(B, S, H, Hkv)
    for _ in range(3):
        A._flash_fwd(q, k, v, True, 1.0 / math.sqrt(128))
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(10):
        A._flash_fwd(q, k, v, True, 1.0 / math.sqrt(128))
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / 10
    flops = 4 * B * H * S * S * 128 / 2
    qh, kh, vh = (t.permute(0, 2, 1, 3) for t in (q, k, v))
    kh, vh = kh.repeat_interleave(4, 1), vh.repeat_interleave(4, 1)
    for _ in range(3):
        torch.nn.functional.scaled_dot_product_attention(qh, kh, vh, is_causal=True)
    e0.record()
    for _ in range(10):
        torch.nn.functional.scaled_dot_product_attention(qh, kh, vh, is_causal=True)
    e1.record()
    torch.cuda.synchronize()
    ms_ref = e0.elapsed_time(e1) / 10
    print(f"flash fwd causal B4 S2048 H16/4: {ms:.3f} ms = {flops / ms / 1e9:.0f} TFLOP/s (torch SDPA {ms_ref:.3f} ms)")
    ops.raise_on_device_error()


@pytest.mark.parametrize("B,S,H,Hkv", [(1, 128, 2, 1), (2, 256, 4, 2), (1, 512, 4, 1), (2, 384, 3, 3), (1, 200, 2, 2),
                                       (1, 1024, 8, 2)])
@pytest.mark.parametrize("causal", [True, False])
def test_flash_backward(B, S, H, Hkv, causal):
    _, q, k, v = _mk(B, S, H, Hkv, seed=1)
    q, k, v = (t.contiguous() for t in (q, k, v))
    scale = 1.0 / math.sqrt(128)
    o, lse = A._flash_fwd(q, k, v, causal, scale)
    do = torch.randn_like(o)
    dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    A._flash_bwd(q, k, v, o, do, lse, dq, dk, dv, causal, scale)
    torch.cuda.synchronize()
    ops.raise_on_device_error()
    qf, kf, vf = (t.float().requires_grad_() for t in (q, k, v))
    ref = ops.sdpa_reference(qf, kf, vf, causal)
    ref.backward(do.float())
    for name, got, want in (("dq", dq, qf.grad), ("dk", dk, kf.grad), ("dv", dv, vf.grad)):
        err = (got.float() - want).abs().max().item()
        lim = 2e-2 * want.abs().max().item() + 2e-2
        assert err <= lim, f"{name}: max err {err} > {lim}"


def test_packed_rope_attention_autograd():
    """RoPE + attention on the packed projection buffer, forward and backward."""
    B, S, H, Hkv, D = 2, 256, 4, 2, 128
    g = torch.Generator(device="cuda").manual_seed(5)
    base = torch.randn(B, S, H + 2 * Hkv, D, device="cuda", generator=g).to(torch.bfloat16)
    cs = ops.rope_table(D, 512, 10000.0, device="cuda")
    x = base.clone().requires_grad_()
    y = A.rope_attention_packed(x * 1.0, cs, None, H, Hkv, causal=True)
    go = torch.randn_like(y)
    y.backward(go)
    xf = base.float().requires_grad_()
    qk = A._rope_torch(xf[:, :, :H + Hkv], cs, None)
    ref = ops.sdpa_reference(qk[:, :, :H], qk[:, :, H:], xf[:, :, H + Hkv:], True)
    ref.backward(go.float())
    assert (y.float() - ref).abs().max().item() < 3e-2
    err = (x.grad.float() - xf.grad).abs().max().item()
    assert err <= 3e-2 * xf.grad.abs().max().item() + 3e-2, err


def test_flash_backward_throughput_report():
    B, S, H, Hkv = 4, 2048, 16, 4
    _, q, k, v = _mk(B, S, H, Hkv)
    q, k, v = (t.contiguous() for t in (q, k, v))
    scale = 1.0 / math.sqrt(128)
    o, lse = A._flash_fwd(q, k, v, True, scale)
    do = torch.randn_like(o)
    dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    for _ in range(3):
        A._flash_bwd(q, k, v, o, do, lse, dq, dk, dv, True, scale)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(10):
        A._flash_bwd(q, k, v, o, do, lse, dq, dk, dv, True, scale)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / 10
    flops = 2.5 * 4 * B * H * S * S * 128 / 2
    print(f"flash bwd causal B4 S2048 H16/4: {ms:.3f} ms = {flops / ms / 1e9:.0f} TFLOP/s (5-GEMM count)")
    ops.raise_on_device_error()


@pytest.mark.parametrize("B,S,H,Hkv", [(4, 2048, 16, 4), (1, 4096, 16, 4)])
def test_flash_forward_backward_at_the_training_shapes(B, S, H, Hkv):
    """The shapes of the 1B configurations (batch 4 x 2048 and a 4096-token sequence, 16 query / 4 KV heads):
    output, log-sum-exp and all three gradients against fp32 attention on the same inputs."""
    qkv, q, k, v = _mk(B, S, H, Hkv, seed=5)
    scale = 1.0 / math.sqrt(128)
    o, lse = A._flash_fwd(q, k, v, True, scale)
    g = torch.Generator(device="cuda").manual_seed(6)
    do = torch.randn(B, S, H, 128, device="cuda", generator=g).to(torch.bfloat16)
    dqkv = torch.empty_like(qkv)
    A._flash_bwd(q, k, v, o, do, lse, dqkv[:, :, :H], dqkv[:, :, H:H + Hkv], dqkv[:, :, H + Hkv:], True, scale)
    torch.cuda.synchronize()
    ops.raise_on_device_error()
    # fp32 oracle, one batch entry at a time (the score matrix of a 4096-token sequence is 1 GB per 16 heads)
    for b in range(B):
        qf, kf, vf = (t[b:b + 1].float().detach().requires_grad_() for t in (q, k, v))
        ref = ops.sdpa_reference(qf, kf, vf, True)
        ref.backward(do[b:b + 1].float())
        assert (o[b:b + 1].float() - ref).abs().max().item() < 2e-2
        for name, got, want in (("dq", dqkv[b:b + 1, :, :H], qf.grad), ("dk", dqkv[b:b + 1, :, H:H + Hkv], kf.grad),
                                ("dv", dqkv[b:b + 1, :, H + Hkv:], vf.grad)):
            err = (got.float() - want).abs().max().item()
            assert err <= 2e-2 * want.abs().max().item() + 2e-2, f"{name}[{b}]: {err}"


@pytest.mark.parametrize("D,H,Hkv", [(64, 24, 4), (32, 4, 2)])
def test_narrow_heads_run_on_the_flash_kernels(D, H, Hkv):
    """Heads narrower than 128 (64 in the reference's benchmark model) take the same kernels zero-padded:
    values and gradients against fp32 attention, and the kernel library is what runs."""
    from khaosz_b200.ops import _lib

    B, S = 2, 512
    g = torch.Generator(device="cuda").manual_seed(7)
    mk = lambda h: torch.randn(B, S, h, D, device="cuda", generator=g).to(torch.bfloat16).requires_grad_()
    q, k, v = mk(H), mk(Hkv), mk(Hkv)
    before = _lib.launch_count()
    out = ops.attention.attention(q, k, v, causal=True)
    assert _lib.launch_count() > before and out.shape == (B, S, H, D)
    do = torch.randn_like(out)
    out.backward(do)
    qf, kf, vf = (t.detach().float().requires_grad_() for t in (q, k, v))
    ref = ops.sdpa_reference(qf, kf, vf, True)
    ref.backward(do.float())
    assert (out.float() - ref).abs().max().item() < 2e-2
    for got, want in ((q.grad, qf.grad), (k.grad, kf.grad), (v.grad, vf.grad)):
        assert (got.float() - want).abs().max().item() <= 2e-2 * want.abs().max().item() + 2e-2


@pytest.mark.parametrize("S,T,H,Hkv,D", [(40, 296, 8, 2, 128), (128, 1024, 4, 4, 128), (200, 333, 6, 3, 64), (1, 130, 8, 2, 128)])
def test_prefill_behind_a_cached_prefix_runs_on_the_flash_kernel(S, T, H, Hkv, D):
    """S new queries against T > S keys (the last S positions of the sequence): causal offset T - S."""
    from khaosz_b200.ops import _lib

    g = torch.Generator(device="cuda").manual_seed(S + T)
    q = torch.randn(2, S, H, D, device="cuda", generator=g).to(torch.bfloat16)
    k = torch.randn(2, T, Hkv, D, device="cuda", generator=g).to(torch.bfloat16)
    v = torch.randn(2, T, Hkv, D, device="cuda", generator=g).to(torch.bfloat16)
    before = _lib.launch_count()
    with torch.inference_mode():
        out = ops.attention.attention(q, k, v, causal=True)
    assert _lib.launch_count() > before
    torch.cuda.synchronize()
    ops.raise_on_device_error()
    ref = ops.sdpa_reference(q.float(), k.float(), v.float(), True)
    assert (out.float() - ref).abs().max().item() < 2e-2
