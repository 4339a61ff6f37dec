"""The allocation-free RMSNorm-backward entry point, called through its exported C symbol.

Some users of the kernel library cannot allocate device memory when they need a kernel (an
arena owner that forbids re-entrant allocation, a latency-critical loop that must not take
the allocator lock, a host that reserved all device memory up front).  For them the library
exports ``kb_rmsnorm_bwd_static``, which keeps its scratch in a fixed device array.  This
test checks it against the regular entry point (which takes the scratch from the caller) on
two consecutive calls with different data, because the shared scratch keeps the previous
call's contents.  The file name makes pytest collect it last.
"""
import ctypes
from ctypes import c_int, c_void_p

import pytest
import torch

pytestmark = pytest.mark.gpu


def _p(t):
    return None if t is None else c_void_p(t.data_ptr())


def _setup_symbol():
    from khaosz_b200.ops import _lib

    handle = _lib.lib()
    fn = handle.kb_rmsnorm_bwd_static
    fn.argtypes = [c_void_p] * 7 + [c_int, c_int, c_void_p]
    fn.restype = c_int
    msg = handle.kb_rmsnorm_bwd_static_error
    msg.restype = ctypes.c_char_p
    return handle, fn, msg


def _case(rows, dim, seed, with_res):
    g = torch.Generator(device="cuda").manual_seed(seed)
    mk = lambda *s: torch.randn(*s, device="cuda", generator=g).to(torch.bfloat16)
    dy, x = mk(rows, dim), mk(rows, dim)
    w = (1 + 0.1 * torch.randn(dim, device="cuda", generator=g)).to(torch.bfloat16)
    dres = mk(rows, dim) if with_res else None
    rstd = torch.rsqrt(x.float().pow(2).mean(-1) + 1e-5)
    return dy, x, w, rstd, dres


def test_static_entry_matches_regular_entry_twice():
    handle, fn, msg = _setup_symbol()
    stream = c_void_p(torch.cuda.current_stream().cuda_stream)
    # the last two cases reach what the small ones do not: more row blocks than the scratch has partial
    # rows (the grid is clamped and each block strides over rows) and the widest supported rows (4096)
    for call, (rows, dim, with_res) in enumerate([(777, 2048, True), (64, 512, False), (5000, 4096, True),
                                                  (5000, 4096, False)]):
        dy, x, w, rstd, dres = _case(rows, dim, 100 + call, with_res)
        # regular entry point: scratch handed in by the caller
        nparts = handle.kb_rmsnorm_bwd_partials(rows)
        partial = torch.empty(nparts, dim, device="cuda", dtype=torch.float32)
        dx_ref, dw_ref = torch.empty_like(x), torch.empty(dim, device="cuda", dtype=torch.float32)
        rc = handle.kb_rmsnorm_bwd(_p(dy), _p(x), _p(w), _p(rstd), _p(dres), _p(dx_ref), _p(dw_ref), _p(partial),
                                   rows, dim, stream)
        assert rc == 0
        # allocation-free entry point: outputs are preallocated here, nothing is allocated inside
        dx, dw = torch.empty_like(x), torch.empty(dim, device="cuda", dtype=torch.float32)
        rc = fn(_p(dy), _p(x), _p(w), _p(rstd), _p(dres), _p(dx), _p(dw), rows, dim, stream)
        assert rc == 0, msg().decode()
        torch.cuda.synchronize()
        err_dx = (dx.float() - dx_ref.float()).abs().max().item()
        assert err_dx <= 2e-2 * dx_ref.float().abs().max().item() + 2e-2
        err_dw = (dw - dw_ref).abs().max().item()
        assert err_dw <= 3e-2 * dw_ref.abs().max().item() + 0.3
        # and both agree with the fp32 PyTorch formula
        xf, wf = x.float().requires_grad_(), w.float().requires_grad_()
        torch.nn.functional.rms_norm(xf, (dim,), wf, 1e-5).backward(dy.float())
        want_dx = xf.grad + (dres.float() if dres is not None else 0)
        assert (dx.float() - want_dx).abs().max().item() <= 2e-2 * want_dx.abs().max().item() + 5e-2
        assert (dw - wf.grad).abs().max().item() <= 3e-2 * wf.grad.abs().max().item() + 0.3


def test_static_entry_rejects_sizes_beyond_its_scratch():
    _, fn, msg = _setup_symbol()
    t = torch.zeros(8, 8192, device="cuda", dtype=torch.bfloat16)
    f = torch.zeros(8192, device="cuda", dtype=torch.float32)
    rc = fn(_p(t), _p(t), _p(t[0]), _p(f), None, _p(t), _p(f), 8, 8192, None)
    assert rc == 4
    assert b"exceeds" in msg()
