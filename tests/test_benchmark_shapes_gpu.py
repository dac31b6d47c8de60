"""Parity at the benchmark's own shapes against the oracle, with the oracle's dense torch ops run on the
device (fp32, TF32 off) because a (T, T) tensor at T = 16384 is 1 GiB.

* whole forward + backward of one sequence at T = 16384, D = 64 and D = 128, bf16: out, dq, dk, dv and the per-key
  totals, shared selection (three heads) and one head per selector, unit-variance inputs and low-scale q, k;
* the reference's CPU case exactly (B = 2, H = 4, T = 1024, D = 64, fp32, seed 0) at the fp32 bar;
* forward rows from a MIDDLE query tile and from the tail, at T = 16384 with all sixteen heads and two
  sequences, and at T = 131072.

Why the low-scale cases: with N(0, 1) inputs the selection a key has received grows by ~0.4 per later
query, so keys more than a few hundred positions back carry weights below 1e-30 and a wrong carry far
back would be invisible.  With q, k ~ N(0, s^2) the selection logit has standard deviation s^2 and the
history term grows by ~0.4 s^2 per query: s = 0.15 keeps every key within ~150 of the top at T = 16384
(tiles a few thousand keys back still matter), s = 0.02 keeps the whole history term below ~3, so every
tile of the sequence contributes at order one.

Bars (relative norm per tensor): bf16 path 2e-2 on outputs and gradients, fp32 path 1e-4.  The achieved
errors are recorded through the ``achieved`` fixture."""

import pytest
import torch

import selective_oracle as oracle
from selective_attention_b200 import _lib, kernels

pytestmark = pytest.mark.gpu


def _rel(got, want):
    return float((got.float() - want.float()).norm() / want.float().norm())


def _inputs(shape, seed, scale_qk=1.0, n=4, dtype=torch.bfloat16):
    g = torch.Generator("cpu").manual_seed(seed)
    ts = [torch.randn(shape, generator=g) for _ in range(n)]
    ts[0] *= scale_qk
    ts[1] *= scale_qk
    return tuple(t.to(dtype) for t in ts)


class _ExactMatmul:
    def __enter__(self):
        self.prev = torch.backends.cuda.matmul.allow_tf32
        torch.backends.cuda.matmul.allow_tf32 = False

    def __exit__(self, *exc):
        torch.backends.cuda.matmul.allow_tf32 = self.prev


@pytest.mark.parametrize("heads", [3, 1])                    # 3: head 0 selects for all; 1: the per-head kernels
@pytest.mark.parametrize("dim,scale_qk", [(64, 1.0), (64, 0.15), (64, 0.02), (128, 1.0), (128, 0.1)])
def test_forward_backward_at_16k_against_the_oracle(heads, dim, scale_qk, achieved):
    seq = 16384
    q, k, v, w = _inputs((1, heads, seq, dim), seed=1000 + heads, scale_qk=scale_qk)
    qq, kk, vv = (t.cuda().requires_grad_(True) for t in (q, k, v))
    out, aux = None, None
    out = kernels.selective_attention(qq, kk, vv)
    out.backward(w.cuda().float())
    with torch.no_grad():
        _, aux = kernels.selective_attention_forward(qq, kk, vv, return_aux=True)
    torch.cuda.synchronize()
    assert _lib.device_status() == 0
    with _ExactMatmul():
        want = oracle.sequence_fwd_bwd(q[0].cuda().float(), k[0].cuda().float(), v[0].cuda().float(),
                                       w[0].cuda().float(), head_chunk=1)
    got = (out.detach()[0], qq.grad[0], kk.grad[0], vv.grad[0])
    errs = {name: _rel(a, b) for name, a, b in zip(("out", "dq", "dk", "dv"), got, want)}
    total_err = float((aux["selected_total"][0] - want[4]).abs().max() / want[4].abs().max().clamp_min(1e-6))
    achieved(f"fwd+bwd T=16384 H={heads} D={dim} bf16 scale_qk={scale_qk}", total_max_rel=total_err, **errs)
    for name, a in zip(("out", "dq", "dk", "dv"), got):
        assert torch.isfinite(a.float()).all(), name
    for name, e in errs.items():
        assert e < 2e-2, (name, e)
    assert total_err < 2e-3


def test_reference_cpu_case_on_the_gpu_fp32(achieved):
    """B = 2, H = 4, T = 1024, D = 64, fp32, q, k, v, dO ~ N(0, 1) from seed 0 in that order."""
    q, k, v, w = _inputs((2, 4, 1024, 64), seed=0, dtype=torch.float32)
    qq, kk, vv = (t.cuda().requires_grad_(True) for t in (q, k, v))
    out = kernels.selective_attention(qq, kk, vv, dot_precision="ieee")
    out.backward(w.cuda())
    torch.cuda.synchronize()
    want = oracle.attention_grads(q, k, v, w)
    got = (out.detach().cpu(), qq.grad.cpu(), kk.grad.cpu(), vv.grad.cpu())
    errs = {name: _rel(a, b) for name, a, b in zip(("out", "dq", "dk", "dv"), got, want)}
    achieved("fwd+bwd B=2 H=4 T=1024 D=64 fp32 (the reference's CPU case)", **errs)
    for name, e in errs.items():
        assert e < 1e-4, (name, e)


@pytest.mark.parametrize("seq,batch,heads,windows,scale_qk", [
    (16384, 2, 16, ((8064, 8320), (16192, 16384)), 1.0),        # across the boundary of query tiles 62 | 63, and the tail
    (16384, 2, 16, ((8064, 8320), (127, 257)), 0.15),
    (16384, 1, 16, ((5000, 5130),), 0.02),
    (131072, 1, 2, ((65472, 65600), (130944, 131072)), 1.0),    # a middle tile boundary and the tail at 131K
    (131072, 1, 2, ((65472, 65600),), 0.008),
])
def test_forward_rows_from_middle_and_tail_tiles(seq, batch, heads, windows, scale_qk, achieved):
    q, k, v = _inputs((batch, heads, seq, 64), seed=seq + heads, scale_qk=scale_qk, n=3)
    qd, kd, vd = q.cuda(), k.cuda(), v.cuda()
    out, aux = kernels.selective_attention_forward(qd, kd, vd, return_aux=True)
    torch.cuda.synchronize()
    assert _lib.device_status() == 0
    assert torch.isfinite(out).all()
    for start, stop in windows:
        with _ExactMatmul():
            rows, want, received = oracle.window_rows(qd.float(), kd.float(), vd.float(), start, stop, chunk=2048)
        got = out[:, :, start:stop]
        err, worst = _rel(got, want), float((got - want).abs().max())
        achieved(f"forward rows [{start}, {stop}) T={seq} B={batch} H={heads} scale_qk={scale_qk}", out=err, max_abs=worst)
        assert err < 2e-2 and worst < 3e-2, (start, stop, err, worst)
        if stop == seq:
            torch.testing.assert_close(aux["selected_total"], received, atol=2e-2, rtol=2e-3)
        elif stop % 128 == 0:
            # the checkpoint at a tile boundary is the selection received from all queries before it
            torch.testing.assert_close(aux["carry"][:, stop // 128, :stop], received, atol=2e-2, rtol=2e-3)
    del out, aux
    torch.cuda.empty_cache()
