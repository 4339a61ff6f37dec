"""Out-of-bounds writes: outputs live inside a sentinel-filled buffer and the guard bands must be
untouched after the kernel (compute-sanitizer is not available on the GPU pool)."""
import pytest
import torch

from khaosz_b200 import ops

pytestmark = pytest.mark.gpu

SENTINEL = 1232.0  # exactly representable in bf16
G = 8              # guard rows / columns (keeps the row pitch a multiple of 16 bytes)


def _guarded(rows, cols):
    buf = torch.full((rows + 2 * G, cols + 2 * G), SENTINEL, device="cuda", dtype=torch.bfloat16)
    return buf, buf[G:G + rows, G:G + cols]


def _guards_intact(buf, rows, cols):
    inner = torch.zeros_like(buf, dtype=torch.bool)
    inner[G:G + rows, G:G + cols] = True
    return bool((buf[~inner] == SENTINEL).all())


@pytest.mark.parametrize("M,N,K,a_mn,b_mn", [(130, 136, 72, False, False), (512, 264, 4096, False, False),
                                             (256, 520, 8192, True, True), (24, 2048, 2048, False, False),
                                             (8192, 2048, 512, False, True)])
def test_gemm_never_writes_outside_its_output(M, N, K, a_mn, b_mn):
    torch.manual_seed(0)
    a = torch.randn((K, M) if a_mn else (M, K), device="cuda").to(torch.bfloat16)
    b = (torch.randn((K, N) if b_mn else (N, K), device="cuda") * 0.05).to(torch.bfloat16)
    buf, out = _guarded(M, N)
    ops.gemm(a, b, a_mn=a_mn, b_mn=b_mn, out=out)
    torch.cuda.synchronize()
    ops.raise_on_device_error()
    assert _guards_intact(buf, M, N)
    ref = (a.float().t() if a_mn else a.float()) @ (b.float() if b_mn else b.float().t())
    assert (out.float() - ref).abs().max().item() <= 2e-2 * ref.abs().max().item() + 2e-2
    # accumulate-into-output epilogue (weight-gradient path) on the same guarded buffer
    before = out.clone()
    ops.gemm(a, b, a_mn=a_mn, b_mn=b_mn, out=out, residual=out)
    torch.cuda.synchronize()
    assert _guards_intact(buf, M, N)
    assert (out.float() - (before.float() + ref)).abs().max().item() <= 3e-2 * ref.abs().max().item() + 3e-2
