"""tcgen05 GEMM vs an fp32 PyTorch product, all operand layouts and ragged shapes."""
import pytest
import torch

from khaosz_b200 import ops

pytestmark = pytest.mark.gpu


def _ref(a, b, a_mn, b_mn, res=None):
    am = a.float().t() if a_mn else a.float()
    bm = b.float() if b_mn else b.float().t()
    out = am @ bm
    if res is not None:
        out = out + res.float()
    return out


def _check(M, N, K, a_mn, b_mn, with_res=False):
    dev = "cuda"
    a = torch.randn((K, M) if a_mn else (M, K), device=dev, dtype=torch.bfloat16)
    b = torch.randn((K, N) if b_mn else (N, K), device=dev, dtype=torch.bfloat16)
    res = torch.randn((M, N), device=dev, dtype=torch.bfloat16) if with_res else None
    out = ops.gemm(a, b, a_mn=a_mn, b_mn=b_mn, residual=res)
    torch.cuda.synchronize()
    ops.raise_on_device_error()
    ref = _ref(a, b, a_mn, b_mn, res)
    err = (out.float() - ref).abs().max().item()
    scale = ref.abs().max().item()
    assert err <= 2e-2 * scale + 1e-2, f"max err {err} (scale {scale}) for {(M, N, K, a_mn, b_mn)}"


@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, True), (True, False)])
@pytest.mark.parametrize("shape", [(128, 256, 64), (256, 512, 256), (384, 768, 1024), (1024, 2048, 512)])
def test_gemm_layouts(shape, a_mn, b_mn):
    _check(*shape, a_mn, b_mn)


@pytest.mark.parametrize("shape", [(200, 264, 72), (8, 2048, 2048), (136, 32000, 128), (4096, 96, 520)])
def test_gemm_ragged(shape):
    _check(*shape, False, False)
    _check(*shape, False, True)
    _check(*shape, True, True)


def test_gemm_residual_and_accumulate():
    _check(512, 1024, 256, False, False, with_res=True)
    a = torch.randn(256, 512, device="cuda", dtype=torch.bfloat16)
    b = torch.randn(256, 384, device="cuda", dtype=torch.bfloat16)
    acc = torch.randn(512, 384, device="cuda", dtype=torch.bfloat16)
    ref = a.float().t() @ b.float() + acc.float()
    ops.gemm(a, b, a_mn=True, b_mn=True, out=acc, residual=acc)
    assert (acc.float() - ref).abs().max().item() <= 2e-2 * ref.abs().max().item() + 1e-2


def test_gemm_many_tiles_persistent():
    # more tiles than SMs: exercises the stage/accumulator phase wrap-around
    _check(2048, 4096, 320, False, False)


def test_linear_autograd_matches_fp32():
    x = torch.randn(4, 96, 256, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    w = torch.randn(512, 256, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    y = ops.linear(x, w)
    g = torch.randn_like(y)
    y.backward(g)
    xf = x.detach().float().requires_grad_()
    wf = w.detach().float().requires_grad_()
    yf = torch.nn.functional.linear(xf, wf)
    yf.backward(g.float())
    for got, ref in ((y, yf), (x.grad, xf.grad), (w.grad, wf.grad)):
        assert (got.float() - ref).abs().max().item() <= 2e-2 * ref.abs().max().item() + 1e-2


def test_gemm_throughput_report():
    """Not an assertion on speed: prints achieved TFLOP/s for the 1B-model shapes."""
    shapes = [(8192, 3072, 2048), (8192, 2048, 2048), (8192, 11264, 2048), (8192, 2048, 5632), (8192, 32000, 2048)]
    for (M, N, K) in shapes:
        a = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
        b = torch.randn(N, K, device="cuda", dtype=torch.bfloat16)
        out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        for _ in range(3):
            ops.gemm(a, b, out=out)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(10):
            ops.gemm(a, b, out=out)
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / 10
        e0.record()
        for _ in range(10):
            torch.matmul(a, b.t(), out=out)
        e1.record()
        torch.cuda.synchronize()
        ms_ref = e0.elapsed_time(e1) / 10
        print(f"GEMM {M}x{N}x{K}: {2 * M * N * K / ms / 1e9:.0f} TFLOP/s (cuBLAS {2 * M * N * K / ms_ref / 1e9:.0f})")
    ops.raise_on_device_error()


@pytest.mark.parametrize("bn", [128, 192, 256])
@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, True)])
def test_gemm_tile_widths(bn, a_mn, b_mn):
    from khaosz_b200.ops._lib import check, lib, ptr, stream

    M, N, K = 1160, 1992, 712
    a = torch.randn((K, M) if a_mn else (M, K), device="cuda", dtype=torch.bfloat16)
    b = torch.randn((K, N) if b_mn else (N, K), device="cuda", dtype=torch.bfloat16)
    r = torch.randn(M, N, device="cuda", dtype=torch.bfloat16)
    out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
    check(lib().kb_gemm_bf16_bn(ptr(a), ptr(b), ptr(out), ptr(r), M, N, K, a.stride(0), b.stride(0), N, N, int(a_mn),
                                int(b_mn), 1, bn, stream()), "gemm_bn")
    torch.cuda.synchronize()
    ops.raise_on_device_error()
    ref = _ref(a, b, a_mn, b_mn, r)
    assert (out.float() - ref).abs().max().item() <= 2e-2 * ref.abs().max().item() + 1e-2


def _pair(a, b, out, r, M, N, K, a_mn, b_mn):
    from khaosz_b200.ops._lib import check, lib, ptr, stream

    check(lib().kb_gemm_bf16_pair(ptr(a), ptr(b), ptr(out), ptr(r), M, N, K, a.stride(0), b.stride(0), out.stride(0),
                                  r.stride(0) if r is not None else 0, int(a_mn), int(b_mn), 1 if r is not None else 0,
                                  stream()), "gemm_pair")


@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, True)])
@pytest.mark.parametrize("shape", [(256, 256, 64), (512, 768, 256), (1160, 1992, 712), (2048, 4096, 320), (136, 520, 2048)])
def test_gemm_cta_pair(shape, a_mn, b_mn):
    M, N, K = shape
    a = torch.randn((K, M) if a_mn else (M, K), device="cuda", dtype=torch.bfloat16)
    b = torch.randn((K, N) if b_mn else (N, K), device="cuda", dtype=torch.bfloat16)
    r = torch.randn(M, N, device="cuda", dtype=torch.bfloat16)
    out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
    _pair(a, b, out, r, M, N, K, a_mn, b_mn)
    torch.cuda.synchronize()
    ops.raise_on_device_error()
    ref = _ref(a, b, a_mn, b_mn, r)
    assert (out.float() - ref).abs().max().item() <= 2e-2 * ref.abs().max().item() + 1e-2


def test_gemm_cta_pair_throughput_report():
    shapes = [(8192, 3072, 2048), (8192, 2048, 2048), (8192, 11264, 2048), (8192, 2048, 5632), (8192, 32000, 2048)]
    for (M, N, K) in shapes:
        a = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
        b = torch.randn(N, K, device="cuda", dtype=torch.bfloat16)
        out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        for _ in range(3):
            _pair(a, b, out, None, M, N, K, False, False)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(10):
            _pair(a, b, out, None, M, N, K, False, False)
        e1.record()
        torch.cuda.synchronize()
        print(f"pair GEMM {M}x{N}x{K}: {2 * M * N * K / (e0.elapsed_time(e1) / 10) / 1e9:.0f} TFLOP/s")
    ops.raise_on_device_error()


@pytest.mark.parametrize("M,N,K", [(4, 2048, 2048), (256, 5632, 2048), (130, 520, 528), (1024, 2048, 5632)])
def test_int8_weight_gemm(M, N, K):
    from khaosz_b200.ops.quant import linear_w8, quantize_w8

    x = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(N, K, device="cuda", dtype=torch.bfloat16) * 0.05
    q, scale = quantize_w8(w)
    q_ref, scale_ref = quantize_w8(w.cpu())
    assert (q.cpu().int() - q_ref.int()).abs().max().item() <= 1 and torch.allclose(scale.cpu(), scale_ref, rtol=1e-3)
    out = linear_w8(x, q, scale)
    torch.cuda.synchronize()
    ops.raise_on_device_error()
    ref = x.float() @ (q.float() * scale[:, None]).t()
    assert (out.float() - ref).abs().max().item() <= 2e-2 * ref.abs().max().item() + 1e-2
    # and the quantisation error itself stays small against the bf16 weights
    full = x.float() @ w.float().t()
    assert (ref - full).abs().max().item() <= 0.05 * full.abs().max().item() + 0.05


@pytest.mark.parametrize("M,N,K", [(128, 256, 128), (512, 1024, 1024), (300, 520, 2048), (8192, 2048, 2048)])
def test_fp8_block_scaled_gemm(M, N, K):
    from khaosz_b200.ops import quant

    x = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    w = (torch.randn(N, K, device="cuda") * 0.05).to(torch.bfloat16)
    a8, sa = quant.quantize_fp8_1x128(x)
    b8, sb = quant.quantize_fp8_128x128(w)
    # quantisers agree with the PyTorch formulation
    a8c, sac = quant.quantize_fp8_1x128(x.cpu())
    assert torch.allclose(sa.cpu(), sac, rtol=1e-5)
    assert (quant.dequantize_fp8(a8.cpu(), sa.cpu(), False) - quant.dequantize_fp8(a8c, sac, False)).abs().max() <= 0.13 * x.abs().max().item()
    b8c, sbc = quant.quantize_fp8_128x128(w.cpu())
    assert torch.allclose(sb.cpu(), sbc, rtol=1e-5)
    out = quant.gemm_fp8(a8, sa, b8, sb)
    torch.cuda.synchronize()
    ops.raise_on_device_error()
    ref = quant.dequantize_fp8(a8, sa, False) @ quant.dequantize_fp8(b8, sb, True).t()
    assert (out.float() - ref).abs().max().item() <= 2e-2 * ref.abs().max().item() + 1e-2
    full = x.float() @ w.float().t()
    assert (ref - full).abs().mean().item() <= 0.05 * full.abs().mean().item() + 1e-3


def test_fp8_linear_autograd_and_throughput():
    from khaosz_b200.ops import quant

    x = torch.randn(256, 1024, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    w = (torch.randn(768, 1024, device="cuda") * 0.05).to(torch.bfloat16).requires_grad_()
    y = quant.linear_fp8(x, w)
    y.sum().backward()
    assert x.grad is not None and w.grad is not None and w.grad.shape == w.shape
    ref = x.detach().float() @ w.detach().float().t()
    assert (y.float() - ref).abs().mean().item() <= 0.06 * ref.abs().mean().item() + 1e-3
    M, N, K = 8192, 11264, 2048
    a = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    b = (torch.randn(N, K, device="cuda") * 0.05).to(torch.bfloat16)
    a8, sa = quant.quantize_fp8_1x128(a)
    b8, sb = quant.quantize_fp8_128x128(b)
    for _ in range(3):
        quant.gemm_fp8(a8, sa, b8, sb)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(10):
        quant.gemm_fp8(a8, sa, b8, sb)
    e1.record()
    torch.cuda.synchronize()
    print(f"fp8 block-scaled GEMM {M}x{N}x{K}: {2 * M * N * K / (e0.elapsed_time(e1) / 10) / 1e9:.0f} TFLOP/s")
    ops.raise_on_device_error()


def test_fp8_input_gradient_of_the_linear_layers():
    """``set_fp8_linear(True, dgrad=True)``: the input gradient of ``ops.linear`` / ``ops.multi_linear`` runs as a
    block-scaled fp8 GEMM over the output gradient and the cached transposed weight image; it must agree with
    the fp32 product to fp8 accuracy, the weight gradient stays the bf16 GEMM, and the cache must follow the
    optimizer's weight generations."""
    from khaosz_b200.ops import functional as Fn

    M, K, N = 512, 1024, 768
    g = torch.Generator(device="cuda").manual_seed(4)
    x = torch.randn(M, K, device="cuda", generator=g).to(torch.bfloat16).requires_grad_()
    w = (torch.randn(N, K, device="cuda", generator=g) * 0.05).to(torch.bfloat16).requires_grad_()
    dy = torch.randn(M, N, device="cuda", generator=g).to(torch.bfloat16)
    Fn.set_fp8_linear(True, dgrad=True)
    try:
        y = ops.linear(x, w)
        y.backward(dy)
        dx_ref = dy.float() @ w.detach().float()
        dw_ref = dy.float().t() @ x.detach().float()
        assert (x.grad.float() - dx_ref).abs().mean().item() <= 0.06 * dx_ref.abs().mean().item() + 1e-3
        assert (w.grad.float() - dw_ref).abs().mean().item() <= 0.01 * dw_ref.abs().mean().item() + 1e-3
        # the kernel product equals the product of the dequantised operands (the GEMM itself is exact to fp32)
        d8, sd = quant_mod().quantize_fp8_1x128(dy)
        w8, sw = Fn._fp8_weight_t(w.detach())
        oracle = quant_mod().dequantize_fp8(d8, sd, False) @ quant_mod().dequantize_fp8(w8, sw, True).t()
        assert (x.grad.float() - oracle).abs().max().item() <= 2e-2 * oracle.abs().max().item()
        # a new weight generation re-quantises the transposed image
        with torch.no_grad():
            w.mul_(2.0)
        Fn.bump_weight_generation()
        x.grad = None
        ops.linear(x, w).backward(dy)
        assert (x.grad.float() - 2 * dx_ref).abs().mean().item() <= 0.06 * (2 * dx_ref).abs().mean().item() + 1e-3
    finally:
        Fn.set_fp8_linear(False)
    ops.raise_on_device_error()


def quant_mod():
    from khaosz_b200.ops import quant

    return quant
