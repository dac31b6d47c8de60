"""Parity at the benchmark's sequence lengths through checks that do not need a (T x T) tensor:
tail rows and per-key totals against the chunked oracle, the two engines against each other, and
linearity of the backward in the cotangent."""

import os

import pytest
import torch

import selective_oracle as oracle
from selective_attention_b200 import _lib, kernels

pytestmark = pytest.mark.gpu


def _inputs(batch, heads, seq, dim, seed, n=3):
    g = torch.Generator("cpu").manual_seed(seed)
    return tuple(torch.randn(batch, heads, seq, dim, generator=g).bfloat16() for _ in range(n))


def _rel(got, want):
    return float((got.float() - want.float()).norm() / want.float().norm())


@pytest.mark.parametrize("seq,tail", [(16384, 192), (131072, 128)])
def test_forward_tail_rows_and_totals_at_benchmark_lengths(seq, tail):
    q, k, v = _inputs(1, 2, seq, 64, seed=seq)
    out, aux = kernels.selective_attention_forward(q.cuda(), k.cuda(), v.cuda(), return_aux=True)
    torch.cuda.synchronize()
    assert _lib.device_status() == 0
    dev = "cuda" if seq > 100_000 else "cpu"               # the oracle's dense torch ops; on the device when long
    prev = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    try:
        rows, want, total = oracle.tail_rows(q.float().to(dev), k.float().to(dev), v.float().to(dev), tail=tail,
                                             chunk=4096)
    finally:
        torch.backends.cuda.matmul.allow_tf32 = prev
    rows, want, total = rows.cpu(), want.cpu(), total.cpu()
    got = out[:, :, rows.cuda()].cpu()
    assert torch.isfinite(out).all()
    assert _rel(got, want) < 2e-2 and (got - want).abs().max() < 3e-2
    torch.testing.assert_close(aux["selected_total"].cpu(), total, atol=2e-2, rtol=2e-3)
    assert aux["selected_total"][0, 0] == 0 and aux["selected_total"][0, -1] == 0      # <BOS> and the last key


def test_tensor_core_and_cuda_core_engines_agree_at_4k():
    q, k, v, w = _inputs(1, 3, 4096, 64, seed=4, n=4)
    results = []
    for engine in ("", "simt"):
        os.environ["SA_B200_ENGINE"] = engine
        try:
            qq, kk, vv = (t.cuda().clone().requires_grad_(True) for t in (q, k, v))
            out = kernels.selective_attention(qq, kk, vv)
            out.backward(w.cuda().float())
            results.append((out.detach(), qq.grad, kk.grad, vv.grad))
        finally:
            os.environ.pop("SA_B200_ENGINE", None)
    torch.cuda.synchronize()
    assert _lib.device_status() == 0
    for name, a, b in zip(("out", "dq", "dk", "dv"), *results):
        assert _rel(a, b) < 2e-2, (name, _rel(a, b))


def test_backward_is_linear_in_the_cotangent_at_16k():
    q, k, v = _inputs(1, 2, 16384, 64, seed=16)
    g = torch.Generator("cpu").manual_seed(99)
    w1, w2 = (torch.randn(1, 2, 16384, 64, generator=g).cuda() for _ in range(2))
    grads = []
    for w in (w1, w2, w1 + w2):
        qq, kk, vv = (t.cuda().clone().requires_grad_(True) for t in (q, k, v))
        kernels.selective_attention(qq, kk, vv).backward(w)
        grads.append((qq.grad.float(), kk.grad.float(), vv.grad.float()))
    torch.cuda.synchronize()
    assert _lib.device_status() == 0
    for name, a, b, both in zip(("dq", "dk", "dv"), *grads):
        assert torch.isfinite(both).all()
        assert _rel(a + b, both) < 2e-2, (name, _rel(a + b, both))


def test_forward_past_the_int32_offset_limit():
    """T = 270,000 (the reference's own long-sequence check, tests/test_selective_kernels.py:333-345): the carry
    of the CUDA-core engine is (1, 8438, 270000) fp32 = 9.1 GB, whose element offsets pass 2^31.  fp32 inputs,
    exact products, head_dim 16; last 1000 rows and the per-key totals against the chunked oracle."""
    seq = 270_000
    if torch.cuda.get_device_properties(0).total_memory < 24 * 2**30:
        pytest.skip("needs a 24 GB GPU")
    g = torch.Generator("cpu").manual_seed(31)
    q, k, v = (torch.randn(1, 2, seq, 16, generator=g).cuda() for _ in range(3))
    got, aux = kernels.selective_attention_forward(q, k, v, dot_precision="ieee", return_aux=True)
    torch.cuda.synchronize()
    assert aux["carry"].numel() > 2**31
    prev = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    try:                                                     # the oracle's dense torch ops, on the device for speed
        rows, want, total = oracle.tail_rows(q, k, v, tail=1000, chunk=8192)
    finally:
        torch.backends.cuda.matmul.allow_tf32 = prev
    torch.testing.assert_close(got[:, :, rows], want, atol=2e-4, rtol=2e-4)
    torch.testing.assert_close(aux["selected_total"], total, atol=1e-2, rtol=1e-3)
    del got, aux
    torch.cuda.empty_cache()
