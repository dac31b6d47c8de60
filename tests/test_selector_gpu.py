"""Head sharding of one sequence: calls that hold some of its heads and a replica of the selection head's rows
(``selector=(q0, k0)``) must reproduce the unsplit call, and their partial selector gradients must add up.
This is the single-process form of the 2-GPU split (each half is what one rank would run)."""

import pytest
import torch

import selective_oracle as oracle
from selective_attention_b200 import _lib, kernels

pytestmark = pytest.mark.gpu


def _rel(got, want):
    return float((got.float() - want.float()).norm() / want.float().norm().clamp_min(1e-12))


def _split_call(q, k, v, w, head_slices, precision):
    """Runs one call per head slice with the selector given separately; returns out, dq, dk, dv of all heads and
    the summed selector gradients."""
    q0 = q[:, 0].detach().clone().requires_grad_(True)
    k0 = k[:, 0].detach().clone().requires_grad_(True)
    outs, dqs, dks, dvs = [], [], [], []
    for hs in head_slices:
        qq, kk, vv = (t[:, hs].detach().clone().requires_grad_(True) for t in (q, k, v))
        out = kernels.selective_attention(qq, kk, vv, dot_precision=precision, selector=(q0, k0))
        out.backward(w[:, hs])
        outs.append(out.detach()); dqs.append(qq.grad); dks.append(kk.grad); dvs.append(vv.grad)
    cat = lambda xs: torch.cat(xs, dim=1)
    return cat(outs), cat(dqs), cat(dks), cat(dvs), q0.grad, k0.grad


@pytest.mark.parametrize("dtype,precision,dim,seq,tol", [
    (torch.float32, "ieee", 32, 300, 1e-4),       # CUDA-core engine
    (torch.bfloat16, None, 64, 700, 2e-2),        # tensor-core engine
    (torch.bfloat16, None, 64, 2049, 2e-2),
    (torch.bfloat16, None, 128, 1000, 2e-2),      # head_dim 128: the split-head-dimension backward with an outside selector
])
def test_two_head_halves_with_a_replicated_selector_equal_the_unsplit_call(dtype, precision, dim, seq, tol, achieved):
    g = torch.Generator("cpu").manual_seed(seq)
    heads = 4
    q, k, v, w = (torch.randn(2, heads, seq, dim, generator=g).to(dtype) for _ in range(4))
    want = oracle.attention_grads(q.float(), k.float(), v.float(), w.float())
    qd, kd, vd, wd = (t.cuda() for t in (q, k, v, w))
    out, dq, dk, dv, dq0, dk0 = _split_call(qd, kd, vd, wd.float(), (slice(0, 2), slice(2, 4)), precision)
    torch.cuda.synchronize()
    assert _lib.device_status() == 0
    # the caller's fold: the summed selector gradients belong to head 0's q and k rows
    dq = dq.float().clone(); dk = dk.float().clone()
    dq[:, 0] += dq0.float()
    dk[:, 0] += dk0.float()
    errs = {n: _rel(a.cpu(), b) for n, a, b in zip(("out", "dq", "dk", "dv"), (out, dq, dk, dv), want)}
    achieved(f"head halves + selector, {dtype} D={dim} T={seq}", **errs)
    for n, e in errs.items():
        assert e < tol, (n, e)
    # and the unsplit call of the same library agrees with the split one to rounding
    qq, kk, vv = (t.clone().requires_grad_(True) for t in (qd, kd, vd))
    ref = kernels.selective_attention(qq, kk, vv, dot_precision=precision)
    ref.backward(wd.float())
    assert _rel(out, ref.detach()) < (1e-6 if dtype == torch.float32 else 1e-3)
    assert _rel(dq, qq.grad) < tol and _rel(dk, kk.grad) < tol


def test_selector_forward_totals_are_identical_on_every_shard():
    g = torch.Generator("cpu").manual_seed(3)
    q, k, v = (torch.randn(1, 6, 500, 64, generator=g).bfloat16().cuda() for _ in range(3))
    sel = (q[:, 0], k[:, 0])
    totals, outs = [], []
    for hs in (slice(0, 2), slice(2, 4), slice(4, 6)):
        out, aux = kernels.selective_attention_forward(q[:, hs], k[:, hs], v[:, hs], return_aux=True, selector=sel)
        totals.append(aux["selected_total"]); outs.append(out)
    whole, aux = kernels.selective_attention_forward(q, k, v, return_aux=True)
    for t in totals:
        torch.testing.assert_close(t, aux["selected_total"], atol=0, rtol=0)
    torch.testing.assert_close(torch.cat(outs, dim=1), whole, atol=1e-5, rtol=1e-5)


def test_one_head_with_an_external_selector_is_not_the_per_head_variant():
    """heads == 1 without a selector means 'this head selects for itself'; with a selector it must not."""
    g = torch.Generator("cpu").manual_seed(4)
    q, k, v = (torch.randn(1, 2, 400, 64, generator=g).bfloat16().cuda() for _ in range(3))
    whole = kernels.selective_attention_forward(q, k, v)
    lone = kernels.selective_attention_forward(q[:, 1:], k[:, 1:], v[:, 1:], selector=(q[:, 0], k[:, 0]))
    torch.testing.assert_close(lone, whole[:, 1:], atol=1e-5, rtol=1e-5)


def test_selector_argument_errors():
    q = torch.randn(1, 2, 64, 64, device="cuda", dtype=torch.bfloat16)
    with pytest.raises(ValueError, match="must all be"):
        kernels.selective_attention_forward(q, q, q, selector=(q[:, 0, :32], q[:, 0]))
    with pytest.raises(ValueError, match="pair"):
        kernels.selective_attention_forward(q, q, q, selector=q)
