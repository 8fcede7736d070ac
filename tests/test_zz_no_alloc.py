"""The workspace-free variant of the adapter-gradient GEMM, called through the C ABI.

Some hosts of this library cannot allocate device memory at the point of the call -- they run
inside a framework that hands them a fixed set of buffers, or in a serving loop where a device
allocation (which can synchronise the GPU) is not tolerated -- so they have no workspace to give to
``k2q_lora_tn``.  ``k2q_lora_tn_static`` keeps the split-T partial sums in a 16 MiB array that is
part of the library image instead.  The array is shared by all calls and keeps the previous call's
contents, hence the second call below with different inputs: stale partial sums must not leak.

This file sorts last on purpose, so that a run that stops at the first failure has already run
every other test.
"""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


def _ptr(t):
    return C.c_void_p(t.data_ptr())


def _both(lib, p, q, scale):
    t, r = p.shape
    c = q.shape[1]
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    ws_bytes = int(lib.k2q_lora_tn_workspace_bytes(t, r, c))
    ws = torch.empty(ws_bytes // 4, dtype=torch.float32, device="cuda")
    ref = torch.full((r, c), float("nan"), device="cuda")
    out = torch.full((r, c), float("nan"), device="cuda")
    rc = lib.k2q_lora_tn(_ptr(p), r, _ptr(q), c, t, r, c, scale, _ptr(ref), c, _ptr(ws), ws_bytes, stream)
    assert rc == 0, lib.k2q_last_error()
    rc = lib.k2q_lora_tn_static(_ptr(p), r, _ptr(q), c, t, r, c, scale, _ptr(out), c, stream)
    assert rc == 0, lib.k2q_last_error()
    torch.cuda.synchronize()
    return out, ref


def test_static_scratch_variant_matches_workspace_variant_twice():
    from k2q import _lib
    lib = _lib.load()
    assert lib.k2q_lora_tn_static_max_bytes() == 16 << 20
    g = torch.Generator().manual_seed(123)
    # first call: a large case (a third of the built-in array)
    p1 = torch.randn(4096, 32, generator=g).cuda()
    q1 = (torch.randn(4096, 3072, generator=g) * 1e-2).to(torch.bfloat16).cuda()
    out1, ref1 = _both(lib, p1, q1, 2.0)
    assert torch.isfinite(out1).all()
    assert torch.allclose(out1, ref1, rtol=2e-4, atol=0.0) and torch.equal(out1, ref1)
    exact = 2.0 * p1.double().t() @ q1.double()
    assert (out1.double() - exact).abs().max() <= 2e-4 * exact.abs().max()
    # second call straight after, smaller and with other data: must not see the first call's sums
    p2 = torch.randn(777, 16, generator=g).cuda()
    q2 = (torch.randn(777, 1536, generator=g) * 1e-2).to(torch.bfloat16).cuda()
    out2, ref2 = _both(lib, p2, q2, -0.5)
    assert torch.allclose(out2, ref2, rtol=2e-4, atol=0.0) and torch.equal(out2, ref2)
    exact2 = -0.5 * p2.double().t() @ q2.double()
    assert (out2.double() - exact2).abs().max() <= 2e-4 * exact2.abs().max()


def test_static_scratch_variant_refuses_oversized_problems():
    from k2q import _lib
    lib = _lib.load()
    t, r, c = 64, 64, 76800                        # one split x 64 x 76800 x 4 B = 19.7 MB > 16 MiB
    assert lib.k2q_lora_tn_workspace_bytes(t, r, c) > lib.k2q_lora_tn_static_max_bytes()
    p = torch.zeros(t, r, device="cuda")
    q = torch.zeros(t, c, dtype=torch.bfloat16, device="cuda")
    out = torch.zeros(r, c, device="cuda")
    rc = lib.k2q_lora_tn_static(_ptr(p), r, _ptr(q), c, t, r, c, 1.0, _ptr(out), c, C.c_void_p(0))
    assert rc == _lib.K2Q_EINVAL
    assert b"built-in array" in lib.k2q_last_error()


def test_static_scratch_variant_allocates_nothing_and_handles_empty_sums():
    """What the entry point is for: after one warm-up call (which resolves the built-in array's address)
    further calls leave the device's free memory and torch's reserved pool exactly as they were.
    T == 0 gives zeros, as the workspace variant does."""
    from k2q import _lib
    lib = _lib.load()
    g = torch.Generator().manual_seed(5)
    p = torch.randn(1024, 16, generator=g).cuda()
    q = (torch.randn(1024, 2048, generator=g) * 1e-2).to(torch.bfloat16).cuda()
    out = torch.empty(16, 2048, device="cuda")
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)

    def call(t_rows):
        rc = lib.k2q_lora_tn_static(_ptr(p), 16, _ptr(q), 2048, t_rows, 16, 2048, 1.0, _ptr(out), 2048, stream)
        assert rc == 0, lib.k2q_last_error()

    call(1024)                                     # warm-up: symbol lookup, kernel attributes
    torch.cuda.synchronize()
    free0, _ = torch.cuda.mem_get_info()
    reserved0 = torch.cuda.memory_reserved()
    for _ in range(3):
        call(1024)
    call(0)
    torch.cuda.synchronize()
    free1, _ = torch.cuda.mem_get_info()
    assert free1 == free0 and torch.cuda.memory_reserved() == reserved0
    assert torch.count_nonzero(out).item() == 0    # the T == 0 call came last
    ref = torch.full((16, 2048), float("nan"), device="cuda")
    rc = lib.k2q_lora_tn(_ptr(p), 16, _ptr(q), 2048, 0, 16, 2048, 1.0, _ptr(ref), 2048, C.c_void_p(0), 0, stream)
    assert rc == 0 and torch.equal(ref, out)
