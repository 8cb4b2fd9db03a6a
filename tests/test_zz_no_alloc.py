"""Allocation-free RMSNorm backward, called through its exported C symbol.

Some callers of this library may not allocate device memory at the moment they call it: code
inside a CUDA-graph capture, code that manages a fixed memory budget by hand, latency-critical
paths that cannot take the allocator's lock.  For them `b200_rmsnorm_bwd_noalloc` keeps its
scratch in a fixed array inside the library.  This test loads the shared object with ctypes (no
torch binding in between), calls the symbol twice in a row on different inputs and checks both
results against the regular entry point, which uses caller-provided scratch.  It lives in its own
file, collected last, and works in a fresh process as well as after the other GPU tests.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _lib():
    from moe_b200.ops import _ext

    _ext.load()  # makes sure the shared object is built and libtorch's CUDA runtime is loaded
    lib = ctypes.CDLL(str(_ext._SO))
    fn = lib.b200_rmsnorm_bwd_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p] * 7 + [ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_void_p]
    lib.b200_rmsnorm_bwd_noalloc_strerror.restype = ctypes.c_char_p
    lib.b200_rmsnorm_bwd_noalloc_strerror.argtypes = [ctypes.c_int]
    return lib


def relerr(a, b):
    a, b = a.float(), b.float()
    return ((a - b).norm() / (b.norm() + 1e-12)).item()


def _inputs(T, H, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    r = lambda *s: torch.randn(*s, device="cuda", generator=g)
    x = r(T, H).bfloat16()
    return dict(dy=r(T, H).bfloat16(), x=x, rstd=torch.rsqrt(x.float().pow(2).mean(-1) + 1e-6).contiguous(),
                w=(1 + 0.1 * r(H)).contiguous(), dres=r(T, H).bfloat16())


def _reference(inp, accumulate_into=None):
    from moe_b200.ops import _ext

    e = _ext.load()
    T, H = inp["x"].shape
    dx = torch.empty_like(inp["x"])
    dw = accumulate_into.clone() if accumulate_into is not None else torch.empty(H, device="cuda")
    part = torch.empty(e.rmsnorm_bwd_blocks(T) * H, device="cuda")
    e.rmsnorm_bwd(inp["dy"], inp["x"], inp["rstd"], inp["w"], inp["dres"], dx, part, dw, accumulate_into is not None)
    return dx, dw


def _noalloc(lib, inp, dw, accumulate):
    T, H = inp["x"].shape
    dx = torch.empty_like(inp["x"])
    stream = torch.cuda.current_stream().cuda_stream
    rc = lib.b200_rmsnorm_bwd_noalloc(inp["dy"].data_ptr(), inp["x"].data_ptr(), inp["rstd"].data_ptr(),
                                      inp["w"].data_ptr(), inp["dres"].data_ptr(), dx.data_ptr(), dw.data_ptr(),
                                      int(accumulate), T, H, ctypes.c_void_p(stream))
    assert rc == 0, lib.b200_rmsnorm_bwd_noalloc_strerror(rc)
    return dx


def test_noalloc_matches_regular_entry_twice_in_a_row():
    lib = _lib()
    # first call (does the one-time set-up on this device), larger problem
    a = _inputs(3000, 1024, seed=1)
    dw_a = torch.full((1024,), 123.0, device="cuda")  # overwritten: accumulate = 0
    dx_a = _noalloc(lib, a, dw_a, accumulate=False)
    # second call right behind it on the same stream: different shape, accumulating into dw.
    # The shared scratch still holds the first call's partial sums; they must not show up here.
    b = _inputs(77, 256, seed=2)
    base = torch.randn(256, device="cuda")
    dw_b = base.clone()
    dx_b = _noalloc(lib, b, dw_b, accumulate=True)
    torch.cuda.synchronize()
    ref_dx_a, ref_dw_a = _reference(a)
    ref_dx_b, ref_dw_b = _reference(b, accumulate_into=base)
    torch.cuda.synchronize()
    assert relerr(dx_a, ref_dx_a) < 1e-6 and relerr(dw_a, ref_dw_a) < 1e-6
    assert relerr(dx_b, ref_dx_b) < 1e-6 and relerr(dw_b, ref_dw_b) < 1e-6
    # and against plain PyTorch, within the tolerance the other kernel tests use
    xh = a["x"].float() * a["rstd"][:, None]
    wdy = a["dy"].float() * a["w"]
    dx_t = a["rstd"][:, None] * (wdy - xh * (wdy * xh).mean(-1, keepdim=True)) + a["dres"].float()
    assert relerr(dx_a, dx_t) < 2e-2 and relerr(dw_a, (a["dy"].float() * xh).sum(0)) < 2e-2


def test_noalloc_rejects_sizes_beyond_its_scratch():
    lib = _lib()
    inp = _inputs(8, 4096, seed=3)  # H above the 2048 limit
    dw = torch.zeros(4096, device="cuda")
    dx = torch.empty_like(inp["x"])
    args = [inp["dy"].data_ptr(), inp["x"].data_ptr(), inp["rstd"].data_ptr(), inp["w"].data_ptr(), None,
            dx.data_ptr(), dw.data_ptr(), 0]
    rc = lib.b200_rmsnorm_bwd_noalloc(*args, 8, 4096, None)
    assert rc == -1 and b"2048" in lib.b200_rmsnorm_bwd_noalloc_strerror(rc)
    assert lib.b200_rmsnorm_bwd_noalloc(*args, 8, 100, None) == -1  # not a multiple of 8
    assert lib.b200_rmsnorm_bwd_noalloc(None, None, None, None, None, None, None, 0, 8, 256, None) == -4
    assert torch.all(dw == 0)  # nothing ran
