"""The bounded waits: a wait that runs out ends its kernel, is reported, and blocks further launches until the
word is cleared.  The wait that runs out here is a probe kernel's wait on an mbarrier nobody arrives on, with a
limit of about a millisecond; it returns by itself and nothing faults."""

import ctypes

import pytest
import torch

import selective_oracle as oracle
from selective_attention_b200 import _lib, kernels

pytestmark = pytest.mark.gpu


def test_a_wait_that_runs_out_is_reported_and_blocks_launches_until_cleared():
    lib = _lib.load()
    g = torch.Generator("cpu").manual_seed(1)
    q, k, v = (torch.randn(1, 2, 300, 64, generator=g).bfloat16().cuda() for _ in range(3))
    want = oracle.attention(q.float().cpu(), k.float().cpu(), v.float().cpu())
    first = kernels.selective_attention_forward(q, k, v)       # creates the mapped timeout flag for this device
    torch.cuda.synchronize()
    assert _lib.device_status() == 0

    _lib.check("sa_selftest_wait_timeout", lib.sa_selftest_wait_timeout(2000, torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()                                   # the probe kernel has returned
    with pytest.raises(_lib.LibraryError, match="DEVICE_TIMEOUT"):
        kernels.selective_attention_forward(q, k, v)
    with pytest.raises(_lib.LibraryError, match="DEVICE_TIMEOUT"):   # and stays refused until someone clears it
        kernels.selective_attention_forward(q, k, v)
    word = _lib.device_status(clear=False)
    assert word == (900 << 8) | 1
    assert _lib.device_status(clear=True) == word
    assert _lib.device_status() == 0

    again = kernels.selective_attention_forward(q, k, v)       # a later launch is not cut short by the old timeout
    torch.cuda.synchronize()
    torch.testing.assert_close(again, first, atol=0, rtol=0)
    assert float((again.cpu() - want).norm() / want.norm()) < 2e-2
    assert _lib.device_status() == 0


def test_probe_limit_is_bounded():
    lib = _lib.load()
    assert lib.sa_selftest_wait_timeout(0, None) == 1
    assert lib.sa_selftest_wait_timeout(10_000_000, None) == 1
