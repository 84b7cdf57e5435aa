"""The allocation-free ghost-norm entry point (``dpk_gram_pair_norm_static``),
called the way its intended users call it: through the C symbol exported by the
shared object, with raw device pointers.

Those users are embedders that may not call ``cudaMalloc`` -- code living inside
another framework's fixed memory plan, host loops that must not block on an
allocator, plug-ins that only ever receive input and output buffers.  The test
checks the symbol against the regular entry point (which takes its scratch
buffer from the caller) on two calls in a row; the second call is smaller than
the first, so anything the first left behind in the shared scratch array would
show up in the second result.

This file sorts last on purpose: a run that stops at the first failure has then
already executed every other test.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _lib():
    from opacus_b200 import _C  # loads torch's libraries and ours

    lib = ctypes.CDLL(_C.__file__)
    fn = lib.dpk_gram_pair_norm_static
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_int,
                   ctypes.c_int, ctypes.c_float, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p,
                   ctypes.c_void_p]
    return _C, fn


def _both(_C, fn, a, g, scale):
    B, T, dx = a.shape
    dg = g.shape[-1]
    dev = a.device
    # regular entry point, scratch from the caller
    w_ref = torch.empty(B, device=dev)
    b_ref = torch.empty(B, device=dev)
    scratch = torch.empty(max(int(_C.gram_pair_scratch_floats(B, T)), 1), device=dev)
    _C.gram_pair_norm(a, None, g, scale, scratch, w_ref, b_ref, False)
    # allocation-free entry point: inputs, outputs, status and stream only
    w = torch.full((B,), -1.0, device=dev)
    b = torch.full((B,), -1.0, device=dev)
    status = torch.zeros(4, dtype=torch.int32, device=dev)
    stream = torch.cuda.current_stream().cuda_stream
    rc = fn(a.data_ptr(), None, g.data_ptr(), B, T, dx, dg, ctypes.c_float(scale), w.data_ptr(), b.data_ptr(), 0,
            status.data_ptr(), ctypes.c_void_p(stream))
    assert rc == 0, f"dpk_gram_pair_norm_static returned cudaError {rc}"
    torch.cuda.synchronize()
    assert int(status[0]) == 0
    return (w, b), (w_ref, b_ref)


def test_static_scratch_entry_point_matches_regular_one():
    _C, fn = _lib()
    dev = torch.device("cuda")
    torch.manual_seed(0)
    # two calls in a row; the second uses fewer work items than the first
    for (B, T, dx, dg) in [(6, 384, 128, 192), (3, 100, 64, 72)]:
        a = torch.randn(B, T, dx, device=dev).bfloat16()
        g = (torch.randn(B, T, dg, device=dev) * 0.1).bfloat16()
        (w, b), (w_ref, b_ref) = _both(_C, fn, a, g, 2.0)
        # same kernel, same item order: the two entry points agree to rounding
        assert torch.allclose(w, w_ref, rtol=1e-6, atol=0), (w, w_ref)
        assert torch.allclose(b, b_ref, rtol=1e-6, atol=0), (b, b_ref)
        # and both agree with the plain fp32 statement within the kernel-test tolerance
        want = torch.bmm(g.float().transpose(1, 2), a.float()).pow(2).sum(dim=(1, 2)) * 2.0
        assert ((w - want).norm() / want.norm()).item() < 2e-3


def test_static_scratch_entry_point_rejects_oversized_problems():
    _C, fn = _lib()
    dev = torch.device("cuda")
    a = torch.zeros(1, 8, 8, device=dev).bfloat16()
    out = torch.zeros(1, device=dev)
    # B * n(n+1)/2 * 2 floats with n = ceil(T/128) exceeds the 2^18-float array; nothing is launched
    rc = fn(a.data_ptr(), None, a.data_ptr(), 4096, 128 * 64, 8, 8, ctypes.c_float(1.0), out.data_ptr(), None, 0, None,
            ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == 1  # cudaErrorInvalidValue
    torch.cuda.synchronize()
