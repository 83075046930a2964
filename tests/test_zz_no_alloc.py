"""The allocation-free RMSNorm backward entry point, called through its exported C symbol.

Some users of the native library cannot call cudaMalloc (code inside a stream capture, plugins with a fixed
memory budget, loops that must not take allocator locks), so the library offers one RMSNorm-backward variant
whose scratch lives in a fixed device array.  This file is named to be collected last: it compares that entry
point with the ordinary one, which takes caller-provided scratch, on two consecutive calls.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _ptr(t):
    return ctypes.c_void_p(t.data_ptr())


def _entry():
    from piper_b200.ops import native

    lib = native.cdll()
    fn = lib.piper_rmsnorm_bwd_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p] * 6 + [ctypes.c_int, ctypes.c_longlong, ctypes.c_int, ctypes.c_void_p]
    err = lib.piper_noalloc_last_error
    err.restype = ctypes.c_char_p
    return fn, err


def _rel(a, b):
    return ((a.float() - b.float()).norm() / (b.float().norm() + 1e-12)).item()


def test_noalloc_rmsnorm_bwd_matches_regular_entry_point_twice():
    from piper_b200.ops import native

    fn, err = _entry()
    ops_c = native.lib()
    dev = torch.device("cuda")
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    for call, (T, D) in enumerate([(1000, 4096), (333, 2048)]):      # second call reuses the dirty scratch
        torch.manual_seed(call)
        x = torch.randn(T, D, device=dev, dtype=torch.bfloat16)
        dy = torch.randn(T, D, device=dev, dtype=torch.bfloat16)
        w = torch.randn(D, device=dev, dtype=torch.bfloat16)
        rstd = torch.rsqrt(x.float().pow(2).mean(-1) + 1e-6)
        # ordinary entry point with caller-provided scratch
        dx_ref = torch.empty_like(x)
        dw_ref = torch.zeros(D, device=dev)
        partial = torch.empty(ops_c.rmsnorm_bwd_num_partials(T) * D, device=dev)
        ops_c.rmsnorm_bwd(dy, x, w, rstd, None, dx_ref, partial, dw_ref, None, False)
        # entry point under test
        dx = torch.empty_like(x)
        dw = torch.full((D,), 7.0, device=dev)                       # must be overwritten, not accumulated
        rc = fn(_ptr(dy), _ptr(x), _ptr(w), _ptr(rstd), _ptr(dx), _ptr(dw), 0, T, D, stream)
        assert rc == 0, err().decode()
        torch.cuda.synchronize()
        assert torch.equal(dx, dx_ref)
        assert _rel(dw, dw_ref) < 1e-6
        # and both agree with the fp32 formula
        xf, dyf, wf = x.float(), dy.float(), w.float()
        xhat = xf * rstd[:, None]
        g = dyf * wf
        want_dx = rstd[:, None] * (g - xhat * (g * xhat).mean(-1, keepdim=True))
        assert _rel(dx, want_dx) < 1e-2
        assert _rel(dw, (dyf * xhat).sum(0)) < 1e-2
        # accumulate mode adds to what is there
        rc = fn(_ptr(dy), _ptr(x), _ptr(w), _ptr(rstd), _ptr(dx), _ptr(dw), 1, T, D, stream)
        assert rc == 0, err().decode()
        torch.cuda.synchronize()
        assert _rel(dw, 2 * dw_ref) < 1e-6


def test_noalloc_rejects_oversized_and_misaligned_shapes():
    fn, err = _entry()
    dev = torch.device("cuda")
    t = torch.zeros(16, device=dev)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    assert fn(_ptr(t), _ptr(t), _ptr(t), _ptr(t), _ptr(t), _ptr(t), 0, 4, 8192 + 8, stream) == -1
    assert b"exceeds" in err()
    assert fn(_ptr(t), _ptr(t), _ptr(t), _ptr(t), _ptr(t), _ptr(t), 0, 4, 12, stream) == -1
    assert b"multiple of 8" in err()
    # more rows than the kernels' 32-bit row index can address: rejected before anything is launched
    assert fn(_ptr(t), _ptr(t), _ptr(t), _ptr(t), _ptr(t), _ptr(t), 0, 2 ** 31, 4096, stream) == -1
    assert b"32-bit" in err()
    torch.cuda.synchronize()
