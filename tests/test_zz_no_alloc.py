"""GPU: the allocation-free backward entry point, flashmhf_backward_static_scratch.

Some hosts of this library cannot supply a workspace and must not cause an allocation while they
run: they handed all device memory to their own planner at start-up, or they bind the C ABI over an
FFI and have no device allocator to pass in (and cudaMalloc/cudaFree would stall the whole device
anyway).  For them the library keeps the dK/dU/dV partial sums in a 72 MiB static device array.  This
test calls that entry point through the C ABI, twice in a row on different inputs (the second,
smaller problem runs over the first call's leftovers in the shared array), and checks each result
against the ordinary flashmhf_backward on the same inputs: both run the same deterministic kernels,
so the results must be equal bit for bit.  It also checks what the entry point is for: across a call
neither the device's free memory nor torch's allocator moves.

Collected last (file name) so that a run stopping at the first failure has already run every other test.
"""
import ctypes as C

import pytest
import torch

from oracle import mhffn_oracle as orc

pytestmark = pytest.mark.gpu


def _static_backward(Q, K, U, V, R, dO, outs=None):
    """The test is the caller: it owns inputs and outputs; the library call itself allocates nothing."""
    from flashmhf_b200 import _lib
    from flashmhf_b200.functional import _dims, _tensor
    lib = _lib.load()
    B, H, S, dh = Q.shape
    hk, E, de, _ = K.shape
    if outs is None:
        outs = [torch.full_like(t, float("nan")) for t in (Q, K, U, V)] + [torch.full_like(R, float("nan"))]
    p = _lib.BwdParams(_dims(B, H, S, dh, hk, E, de, Q.dtype), _tensor(Q), _tensor(K), _tensor(U), _tensor(V),
                       _tensor(R), _tensor(dO), *[_tensor(t) for t in outs], None, 0,   # no workspace passed
                       _lib.Scaling(1.0, 1.0, 1.0), 0)
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    free0, alloc0, reserved0 = torch.cuda.mem_get_info()[0], torch.cuda.memory_allocated(), torch.cuda.memory_reserved()
    rc = lib.flashmhf_backward_static_scratch(C.byref(p), stream)
    torch.cuda.synchronize()
    moved = (torch.cuda.mem_get_info()[0] - free0, torch.cuda.memory_allocated() - alloc0,
             torch.cuda.memory_reserved() - reserved0)
    _lib.check(rc)
    _lib.device_status()
    return outs, moved


def test_static_scratch_matches_workspace_entry_point_two_calls_in_a_row():
    import flashmhf_b200 as fm
    from flashmhf_b200 import _lib
    shapes = [(2, 4, 2, 640, 128, 3, 128),   # several token tiles per split, shared K/U/V heads
              (1, 2, 2, 200, 96, 2, 64)]     # smaller, ragged, different head dim: reuses a dirty array
    for i, (B, H, Hk, S, dh, E, de) in enumerate(shapes):
        ins = [t.cuda() for t in orc.make_op_inputs(B, H, S, dh, E, de, Hkuv=Hk, seed=40 + i, dtype=torch.bfloat16)]
        d = _lib.Dims(B, H, S, dh, Hk, E, de, _lib.BF16)
        assert 0 < _lib.load().flashmhf_backward_workspace_bytes(C.byref(d)) <= _lib.STATIC_SCRATCH_BYTES
        want = fm.backward_raw(*ins)
        got, _ = _static_backward(*ins)            # on a device's first call this also looks up the array's address
        for name, a, b in zip("dQ dK dU dV dR".split(), got, want):
            assert torch.isfinite(a.float()).all(), name
            assert torch.equal(a, b), (i, name)
        # once more into the same output buffers: the call must leave the device's memory exactly as it found it
        again, moved = _static_backward(*ins, outs=got)
        assert moved == (0, 0, 0), f"free / allocated / reserved bytes moved by {moved}"
        for name, a, b in zip("dQ dK dU dV dR".split(), again, want):
            assert torch.equal(a, b), (i, name)


def test_static_scratch_refuses_oversized_and_check_mode():
    from flashmhf_b200 import _lib
    from flashmhf_b200.functional import _tensor
    lib = _lib.load()
    # the 1.3B layer's weights (16 heads x 5632 x 128): 138 MB of partial sums per split -> over the limit
    d = _lib.Dims(1, 16, 128, 128, 16, 22, 256, _lib.BF16)
    assert lib.flashmhf_backward_workspace_bytes(C.byref(d)) > _lib.STATIC_SCRATCH_BYTES
    x = torch.zeros(16, device="cuda", dtype=torch.bfloat16)   # never read: the size check comes first
    t = _tensor(x.view(1, 1, 1, 16))
    p = _lib.BwdParams(d, *[t] * 11, None, 0, _lib.Scaling(1.0, 1.0, 1.0), 0)
    assert lib.flashmhf_backward_static_scratch(C.byref(p), None) == -10
    assert b"72 MiB" in lib.flashmhf_strerror(-10)
    p.d.dtype = _lib.F32_CHECK
    assert lib.flashmhf_backward_static_scratch(C.byref(p), None) == -3
