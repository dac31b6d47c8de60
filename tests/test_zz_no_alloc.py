"""The allocation-free forward entry point (library-owned scratch) against the ordinary forward.

Some callers cannot allocate device memory at call time: a serving loop whose memory was all handed to
a cache pool at start-up, or a bare C host that only holds the buffers it was given.  For them the
library keeps the forward's scratch (the running-selection checkpoints) in a fixed device array.  This
test drives that entry point through the C ABI exactly as such a caller would (raw pointers, no torch
allocation between the two calls) and checks that it returns what sa_forward returns: bit for bit,
since the same kernels run, on two calls in a row with different shapes so that stale scratch contents
from the first call are in place during the second."""

import ctypes

import pytest
import torch

from selective_attention_b200 import _lib, kernels

pytestmark = pytest.mark.gpu


def _problem(q, k, v, engine):
    return kernels._problem(q, k, v, engine, exempt=1)


def _both_forwards(lib, q, k, v, engine, bufs):
    out_a, lse_a, tot_a, out_b, lse_b, tot_b, carry = bufs
    prob = _problem(q, k, v, engine)
    stream = torch.cuda.current_stream().cuda_stream
    _lib.check("sa_forward", lib.sa_forward(ctypes.byref(prob), q.data_ptr(), k.data_ptr(), v.data_ptr(),
                                            out_a.data_ptr(), lse_a.data_ptr(), carry.data_ptr(), tot_a.data_ptr(),
                                            stream))
    _lib.check("sa_forward_static_scratch",
               lib.sa_forward_static_scratch(ctypes.byref(prob), q.data_ptr(), k.data_ptr(), v.data_ptr(),
                                             out_b.data_ptr(), lse_b.data_ptr(), tot_b.data_ptr(), stream))


@pytest.mark.parametrize("engine,dtype,dim", [(_lib.ENGINE_TCGEN05, torch.bfloat16, 64),
                                              (_lib.ENGINE_SIMT, torch.float32, 32)])
def test_static_scratch_forward_equals_the_ordinary_forward_twice_in_a_row(engine, dtype, dim):
    lib = _lib.load()
    gen = torch.Generator("cpu").manual_seed(17)
    shapes = [(2, 3, 700, dim), (1, 2, 130, dim)]          # the second call sees the first call's leftovers
    inputs = [tuple(torch.randn(s, generator=gen).to(dtype).cuda() for _ in range(3)) for s in shapes]
    # every buffer of both calls exists before the first call: nothing is allocated in between
    bufs = []
    for (b, h, t, d) in shapes:
        mk = lambda *shape: torch.full(shape, float("nan"), device="cuda")
        bufs.append((mk(b, h, t, d), mk(b, h, t), mk(b, t), mk(b, h, t, d), mk(b, h, t), mk(b, t),
                     mk(b, lib.sa_carry_checkpoints(engine, t), t)))
    torch.cuda.synchronize()
    before = torch.cuda.memory_stats()["allocation.all.allocated"]
    for (q, k, v), buf in zip(inputs, bufs):
        _both_forwards(lib, q, k, v, engine, buf)
    assert torch.cuda.memory_stats()["allocation.all.allocated"] == before
    torch.cuda.synchronize()
    assert _lib.device_status() == 0
    for buf in bufs:
        out_a, lse_a, tot_a, out_b, lse_b, tot_b, _ = buf
        assert torch.isfinite(out_b).all()
        torch.testing.assert_close(out_b, out_a, atol=0, rtol=0)
        torch.testing.assert_close(lse_b, lse_a, atol=0, rtol=0)
        torch.testing.assert_close(tot_b, tot_a, atol=0, rtol=0)


def test_static_scratch_rejects_problems_beyond_its_capacity():
    lib = _lib.load()
    cap = lib.sa_static_scratch_floats()
    assert cap == 2 * 1024 * 1024
    q = torch.zeros(1, 1, 20000, 64, dtype=torch.bfloat16, device="cuda")     # 158 checkpoints x 20000 keys > capacity
    out = torch.empty(1, 1, 20000, 64, device="cuda")
    lse = torch.empty(1, 1, 20000, device="cuda")
    tot = torch.empty(1, 20000, device="cuda")
    prob = _problem(q, q, q, _lib.ENGINE_TCGEN05)
    status = lib.sa_forward_static_scratch(ctypes.byref(prob), q.data_ptr(), q.data_ptr(), q.data_ptr(), out.data_ptr(),
                                           lse.data_ptr(), tot.data_ptr(), None)
    assert status == 7 and lib.sa_status_string(status) == b"problem exceeds the fixed capacity"
    with pytest.raises(_lib.LibraryError, match="TOO_LARGE"):
        _lib.check("sa_forward_static_scratch", status)
