"""Leaving out dead tiles (``skip_dead_tiles=True``): (query tile, key tile) pairs whose probabilities are all exactly
zero are not computed.  The results must be those of the full computation: the forward bit for bit, the gradients up
to the order of the fp32 reductions, and both within the usual bar of the oracle."""

import pytest
import torch

import selective_oracle as oracle
from selective_attention_b200 import _lib, kernels

pytestmark = pytest.mark.gpu


def _inputs(batch, heads, seq, dim, seed, scale_qk=1.0):
    g = torch.Generator("cpu").manual_seed(seed)
    q, k, v, w = (torch.randn(batch, heads, seq, dim, generator=g) for _ in range(4))
    return (q * scale_qk).bfloat16(), (k * scale_qk).bfloat16(), v.bfloat16(), w.bfloat16()


def _rel(a, b):
    return float((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-30))


def _lower(live):
    """The entries of the table that mean something: key tile <= query tile."""
    nt = live.shape[-1]
    mask = torch.tril(torch.ones(nt, nt, dtype=torch.bool, device=live.device))
    return live[:, mask]


def _run(q, k, v, w, skip, exempt=1):
    qq, kk, vv = (t.cuda().requires_grad_(True) for t in (q, k, v))
    out = kernels.selective_attention(qq, kk, vv, exempt=exempt, skip_dead_tiles=skip)
    out.backward(w.cuda().float())
    torch.cuda.synchronize()
    assert _lib.device_status() == 0
    return out.detach(), qq.grad, kk.grad, vv.grad


@pytest.mark.parametrize("heads,dim,seq", [(3, 64, 2049), (1, 64, 1500), (2, 128, 2049), (1, 128, 1300)])
def test_results_equal_the_full_computation_when_most_far_tiles_are_dead(heads, dim, seq, achieved):
    q, k, v, w = _inputs(2, heads, seq, dim, seed=seq + heads)
    with torch.no_grad():
        full, aux_full = kernels.selective_attention_forward(q.cuda(), k.cuda(), v.cuda(), return_aux=True)
        before = _lib.launch_count()
        lean, aux = kernels.selective_attention_forward(q.cuda(), k.cuda(), v.cuda(), return_aux=True, skip_dead_tiles=True)
        assert _lib.launch_count() - before == 5          # colsum, scan, tile norms, tile table, forward
    live = _lower(aux["live_tiles"])
    nt = (seq + 127) // 128
    frac = float((live != 0).float().mean())
    achieved(f"live tiles T={seq} H={heads} D={dim} N(0,1)", live_fraction=frac)
    assert frac < 0.9                                      # unit-variance q, k: keys ~500 positions back are dead
    assert bool((aux["live_tiles"][:, torch.arange(nt), torch.arange(nt)] != 0).all())   # the diagonal is always computed
    assert bool((aux["live_tiles"][:, :, 0] != 0).all())  # key tile 0 holds the exempt <BOS> key: never dead
    assert torch.equal(lean, full)
    assert torch.equal(aux["rmax"], aux_full["rmax"]) and torch.equal(aux["selected_total"], aux_full["selected_total"])

    got = _run(q, k, v, w, skip=True)
    ref = _run(q, k, v, w, skip=False)
    assert torch.equal(got[0], ref[0])
    for name, a, b in zip(("dq", "dk", "dv"), got[1:], ref[1:]):
        assert _rel(a, b) < 2e-3, (name, _rel(a, b))       # the order of the fp32 reductions only
    want = oracle.attention_grads(q.float(), k.float(), v.float(), w.float())
    for name, a, b in zip(("out", "dq", "dk", "dv"), got, want):
        assert _rel(a.cpu(), b) < 2e-2, (name, _rel(a.cpu(), b))


def test_nothing_is_left_out_when_the_selection_is_weak():
    q, k, v, w = _inputs(1, 2, 1500, 64, seed=5, scale_qk=0.05)
    with torch.no_grad():
        full = kernels.selective_attention_forward(q.cuda(), k.cuda(), v.cuda())
        lean, aux = kernels.selective_attention_forward(q.cuda(), k.cuda(), v.cuda(), return_aux=True, skip_dead_tiles=True)
    assert bool((_lower(aux["live_tiles"]) != 0).all())
    assert torch.equal(lean, full)


def test_exempt_prefix_keeps_its_key_tiles_alive():
    q, k, v, w = _inputs(1, 2, 2049, 64, seed=6)
    with torch.no_grad():
        _, aux = kernels.selective_attention_forward(q.cuda(), k.cuda(), v.cuda(), return_aux=True, exempt=200,
                                                     skip_dead_tiles=True)
    live = aux["live_tiles"]
    assert bool((live[:, :, 0] != 0).all())
    assert bool((live[:, 1:, 1] != 0).all())               # keys 128..199 are exempt too
    assert not bool((_lower(live) != 0).all())
    got = _run(q, k, v, w, skip=True, exempt=200)
    want = oracle.attention_grads(q.float(), k.float(), v.float(), w.float(), exempt=200)
    for name, a, b in zip(("out", "dq", "dk", "dv"), got, want):
        assert _rel(a.cpu(), b) < 2e-2, (name, _rel(a.cpu(), b))


def test_head_halves_with_a_replicated_selector():
    q, k, v, w = _inputs(1, 4, 1800, 64, seed=8)
    ref = _run(q, k, v, w, skip=False)
    outs, dqs = [], []
    q0 = q[:, 0].cuda().requires_grad_(True)
    k0 = k[:, 0].cuda().requires_grad_(True)
    for hs in (slice(0, 2), slice(2, 4)):
        qq, kk, vv = (t[:, hs].cuda().requires_grad_(True) for t in (q, k, v))
        out = kernels.selective_attention(qq, kk, vv, selector=(q0, k0), skip_dead_tiles=True)
        out.backward(w[:, hs].cuda().float())
        outs.append(out.detach())
        dqs.append(qq.grad)
    torch.cuda.synchronize()
    assert _lib.device_status() == 0
    assert torch.equal(torch.cat(outs, 1), ref[0])
    dq = torch.cat(dqs, 1).float()
    dq[:, 0] += q0.grad.float()
    assert _rel(dq, ref[1]) < 1e-2


def test_packed_projection_form():
    g = torch.Generator("cpu").manual_seed(11)
    b, t, h, d = 1, 1700, 2, 64
    qkv = torch.randn(b, t, 3, h, d, generator=g).bfloat16().cuda()
    w = torch.randn(b, t, h * d, generator=g).bfloat16().cuda()
    res = []
    for skip in (True, False):
        x = qkv.clone().requires_grad_(True)
        y = kernels.selective_attention_packed(x, skip_dead_tiles=skip)
        y.backward(w)
        res.append((y.detach(), x.grad))
    torch.cuda.synchronize()
    assert _lib.device_status() == 0
    assert torch.equal(res[0][0], res[1][0])
    assert _rel(res[0][1], res[1][1]) < 2e-3


@pytest.mark.parametrize("first,second,per_head", [(1536, 700, False), (1300, 1000, False), (1100, 900, True)])
def test_chunked_prefill_skips_the_dead_part_of_the_cache(first, second, per_head):
    """A continued prefill with the option on returns the rows and the per-key selection of one without, bit for bit."""
    from selective_attention_b200 import mixers
    g = torch.Generator("cpu").manual_seed(first + second)
    total, heads = first + second, 2
    q, k, v = (torch.randn(1, heads, total, 64, generator=g).bfloat16().cuda() for _ in range(3))
    rows, sels = [], []
    for skip in (False, True):
        slot = mixers.SelectiveAttentionSlot(n_heads=heads, context_length=total + 8, per_head=per_head)
        _, cache = slot.begin_cache(q[:, :, :first], k[:, :, :first], v[:, :, :first])
        before = _lib.launch_count()
        rows.append(slot.extend_cache(q[:, :, first:], k[:, :, first:], v[:, :, first:], cache, skip_dead_tiles=skip))
        assert _lib.launch_count() - before == (5 if skip else 3)      # + tile norms, tile table
        sels.append(cache["selected"].clone())
    torch.cuda.synchronize()
    assert _lib.device_status() == 0
    assert torch.equal(rows[0], rows[1]) and torch.equal(sels[0], sels[1])


@pytest.mark.parametrize("heads,per_head,dim", [(4, False, 64), (2, False, 128), (3, True, 64)])
def test_decode_leaves_out_the_dead_part_of_the_cache(heads, per_head, dim):
    """Decode steps on a cache with key norms (dead 64-key stages are not read) against the same steps without:
    outputs and the history vector must be identical.  With one selector per head every CTA stays dense."""
    import math
    from selective_attention_b200 import mixers
    g = torch.Generator("cpu").manual_seed(17 + heads)
    t0, steps = 6000, 5
    q, k, v = (torch.randn(1, heads, t0 + steps, dim, generator=g).bfloat16().cuda() for _ in range(3))
    outs, sels = [], []
    for live in (False, True):
        slot = mixers.SelectiveAttentionSlot(n_heads=heads, context_length=t0 + 16, per_head=per_head)
        _, cache = slot.begin_cache(q[:, :, :t0], k[:, :, :t0], v[:, :, :t0], live_keys=live)
        if live and not per_head:                     # the case must have something to leave out: head 1, first step
            sel = cache["selected"][0, 0, :t0].float()
            kn = cache["key_norms"][0, 1, :t0]
            q1 = q[0, 1, t0].float()
            c1 = math.log2(math.e) / math.sqrt(dim)
            z_new = float((q1 * k[0, 1, t0].float()).sum()) * c1
            alive = c1 * q1.norm() * kn - math.log2(math.e) * sel >= z_new - 150
            stages = alive[: t0 // 64 * 64].view(-1, 64).any(dim=1)
            assert float(stages.float().mean()) < 0.5
        ys = [slot.step_cache(q[:, :, t0 + s:t0 + s + 1], k[:, :, t0 + s:t0 + s + 1], v[:, :, t0 + s:t0 + s + 1], cache)
              for s in range(steps)]
        outs.append(torch.cat(ys, dim=2))
        sels.append(cache["selected"].clone())
        if live:
            want = kernels.key_norms(cache["k"][:, :, :t0 + steps])
            torch.testing.assert_close(cache["key_norms"][:, :, :t0 + steps], want, atol=1e-3, rtol=1e-3)
    torch.cuda.synchronize()
    assert _lib.device_status() == 0
    assert torch.equal(outs[0], outs[1])
    assert torch.equal(sels[0], sels[1])


def test_unsupported_engines_ignore_the_request():
    g = torch.Generator("cpu").manual_seed(1)
    q, k, v = (torch.randn(1, 2, 200, 32, generator=g).cuda() for _ in range(3))
    a = kernels.selective_attention_forward(q, k, v, skip_dead_tiles=True)
    b = kernels.selective_attention_forward(q, k, v)
    assert torch.equal(a, b)
