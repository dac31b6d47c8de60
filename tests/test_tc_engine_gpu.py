"""Tensor-core (tcgen05) engine against the CPU oracle on bf16-rounded inputs.

Tolerances: the bf16 bar is 2e-2 (relative norm) on outputs and gradients; the selection totals and the
carry come from fp32 accumulators of bf16 products and are held to 1e-3."""

import pytest
import torch

import selective_oracle as oracle
from selective_attention_b200 import _lib, kernels

pytestmark = pytest.mark.gpu


def _inputs(batch, heads, seq, dim, seed, scale=1.0, n=4):
    g = torch.Generator("cpu").manual_seed(seed)
    return tuple((scale * torch.randn(batch, heads, seq, dim, generator=g)).bfloat16() for _ in range(n))


def _rel(got, want):
    """Relative norm error; the floor keeps tensors that are analytically zero (T = 1 gradients of q, k)
    from turning rounding noise into a ratio."""
    floor = 1e-3 * want.numel() ** 0.5
    return float((got.float() - want).norm() / want.norm().clamp_min(floor))


@pytest.mark.parametrize("seq", [1, 2, 63, 64, 65, 128, 129, 300, 1000, 2049])
@pytest.mark.parametrize("dim,scale", [(64, 1.0), (64, 0.3), (128, 0.5)])
def test_forward_matches_oracle(seq, dim, scale):
    heads = 3
    q, k, v, _ = _inputs(2, heads, seq, dim, seed=seq + dim, scale=scale)
    out, aux = kernels.selective_attention_forward(q.cuda(), k.cuda(), v.cuda(), return_aux=True)
    torch.cuda.synchronize()
    assert _lib.device_status() == 0
    assert aux["carry_m"] == 128
    want = oracle.attention(q.float(), k.float(), v.float())
    assert _rel(out.cpu(), want) < 2e-2, _rel(out.cpu(), want)
    assert (out.cpu() - want).abs().max() < 3e-2
    total = oracle.selected_total(q.float(), k.float())[:, 0]
    torch.testing.assert_close(aux["selected_total"].cpu(), total, atol=1e-3, rtol=1e-3)
    # carry row r = selection received from queries < 128 r
    sel = oracle.selection_matrix(q[:, 0].float(), k[:, 0].float())
    for r in range(aux["carry"].shape[1]):
        want_row = sel[:, : 128 * r].sum(dim=1)
        got_row = aux["carry"][:, r].cpu()
        valid = torch.arange(seq) < 128 * (r + 1)          # keys past the tile are never read
        torch.testing.assert_close(got_row[:, valid], want_row[:, valid], atol=1e-3, rtol=1e-3)


@pytest.mark.parametrize("seq", [1, 130, 777])
@pytest.mark.parametrize("dim", [64, 128])
def test_forward_one_head_per_selector(seq, dim):
    """heads == 1 (the per-head form) runs the kernels' own-logits instantiation, which at head_dim 128 also has its
    own load schedule (one K tile in shared memory serves both the selection and the attention logits)."""
    q, k, v, _ = _inputs(3, 1, seq, dim, seed=seq + dim + 1, scale=0.7)
    out, aux = kernels.selective_attention_forward(q.cuda(), k.cuda(), v.cuda(), return_aux=True, exempt=2)
    torch.cuda.synchronize()
    assert _lib.device_status() == 0
    want = oracle.attention(q.float(), k.float(), v.float(), exempt=2)
    assert _rel(out.cpu(), want) < 2e-2, _rel(out.cpu(), want)
    torch.testing.assert_close(aux["selected_total"].cpu(), oracle.selected_total(q.float(), k.float(), 2)[:, 0],
                               atol=1e-3, rtol=1e-3)


def test_forward_head_dim_128_strided_views_and_exempt():
    b, t, h, d = 2, 300, 3, 128
    g = torch.Generator("cpu").manual_seed(11)
    packed = (0.5 * torch.randn(b, t, 3, h, d, generator=g)).bfloat16().cuda()   # fused QKV projection layout
    q, k, v = (packed[:, :, i].transpose(1, 2) for i in range(3))
    assert not q.is_contiguous()
    out = kernels.selective_attention_forward(q, k, v, exempt=40)
    want = oracle.attention(q.float().cpu(), k.float().cpu(), v.float().cpu(), exempt=40)
    assert _rel(out.cpu(), want) < 2e-2


@pytest.mark.parametrize("exempt", [3, 16, 70, 200])
def test_forward_exempt_prefix(exempt):
    q, k, v, _ = _inputs(1, 2, 333, 64, seed=exempt)
    out, aux = kernels.selective_attention_forward(q.cuda(), k.cuda(), v.cuda(), return_aux=True, exempt=exempt)
    want = oracle.attention(q.float(), k.float(), v.float(), exempt=exempt)
    assert _rel(out.cpu(), want) < 2e-2
    torch.testing.assert_close(aux["selected_total"].cpu(), oracle.selected_total(q.float(), k.float(), exempt)[:, 0],
                               atol=1e-3, rtol=1e-3)


def test_forward_takes_strided_views_without_a_copy():
    b, h, t, d = 2, 4, 260, 64
    g = torch.Generator("cpu").manual_seed(5)
    packed = torch.randn(b, t, 3, h, d, generator=g).bfloat16().cuda()       # fused QKV projection layout
    q, k, v = (packed[:, :, i].transpose(1, 2) for i in range(3))
    assert not q.is_contiguous()
    out = kernels.selective_attention_forward(q, k, v)
    want = oracle.attention(q.float().cpu(), k.float().cpu(), v.float().cpu())
    assert _rel(out.cpu(), want) < 2e-2


def _fwd_bwd(q, k, v, w, **kw):
    qq, kk, vv = (t.cuda().clone().requires_grad_(True) for t in (q, k, v))
    out = kernels.selective_attention(qq, kk, vv, **kw)
    (out * w.cuda().float()).sum().backward()
    torch.cuda.synchronize()
    assert _lib.device_status() == 0
    return out.detach().cpu(), qq.grad.cpu(), kk.grad.cpu(), vv.grad.cpu()


@pytest.mark.parametrize("seq", [1, 2, 64, 65, 128, 129, 300, 1000, 2049])
@pytest.mark.parametrize("heads,scale", [(1, 1.0), (3, 1.0), (4, 0.3)])
@pytest.mark.parametrize("dim", [64, 128])
def test_backward_matches_oracle(seq, heads, scale, dim):
    q, k, v, w = _inputs(2, heads, seq, dim, seed=seq + heads, scale=scale)
    before = _lib.launch_count()
    got = _fwd_bwd(q, k, v, w)
    assert _lib.launch_count() - before == 3 + 4          # colsum, scan, forward | dbar, backward, 2 x fold
    want = oracle.attention_grads(q.float(), k.float(), v.float(), w.float())
    for name, a, b in zip(("out", "dq", "dk", "dv"), got, want):
        assert a.dtype == (torch.float32 if name == "out" else torch.bfloat16)
        assert torch.isfinite(a.float()).all(), name
        assert _rel(a, b) < 2e-2, (name, _rel(a, b))


def test_backward_selection_gradient_only_through_history():
    q, k, v, _ = _inputs(1, 3, 200, 64, seed=3, scale=1.0)
    w = torch.ones(1, 3, 200, 64)
    w[:, 0] = 0
    _, dq, dk, dv = _fwd_bwd(q, k, v, w)
    _, rq, rk, rv = oracle.attention_grads(q.float(), k.float(), v.float(), w)
    assert rq[:, 0].abs().max() > 1e-4 and dv[:, 0].float().abs().max() == 0
    for a, b in ((dq, rq), (dk, rk), (dv, rv)):
        assert _rel(a, b) < 2e-2


@pytest.mark.parametrize("heads", [1, 2])                  # one head per selector runs the merged-gradient kernel
@pytest.mark.parametrize("exempt", [3, 70, 200])
def test_backward_exempt_prefix(exempt, heads):
    q, k, v, w = _inputs(1, heads, 333, 64, seed=exempt)
    got = _fwd_bwd(q, k, v, w, exempt=exempt)
    want = oracle.attention_grads(q.float(), k.float(), v.float(), w.float(), exempt=exempt)
    for name, a, b in zip(("out", "dq", "dk", "dv"), got, want):
        assert _rel(a, b) < 2e-2, (name, _rel(a, b))


@pytest.mark.parametrize("heads", [1, 3])
def test_head_dim_128_backward_exempt_prefix_and_selection_only_gradient(heads):
    """head_dim 128: two CTAs per (head, key tile), one per half of the head dimension; the query-side gradients
    leave transposed.  An exempt prefix past the first key tile, and a cotangent that is zero on the selection head
    so that its q / k gradients come only through the other heads' history terms."""
    q, k, v, w = _inputs(1, heads, 333, 128, seed=50 + heads, scale=0.8)
    if heads > 1:
        w[:, 0] = 0
    got = _fwd_bwd(q, k, v, w, exempt=140)
    want = oracle.attention_grads(q.float(), k.float(), v.float(), w.float(), exempt=140)
    for name, a, b in zip(("out", "dq", "dk", "dv"), got, want):
        assert _rel(a, b) < 2e-2, (name, _rel(a, b))


def test_reference_layout_of_the_carry_on_request():
    """aux["carry"] every 32 queries (the reference's CARRY_M) from the bf16 path, zero where nothing is stored."""
    q, k, v, _ = _inputs(2, 2, 300, 64, seed=21)
    _, native = kernels.selective_attention_forward(q.cuda(), k.cuda(), v.cuda(), return_aux=True)
    _, aux = kernels.selective_attention_forward(q.cuda(), k.cuda(), v.cuda(), return_aux=True, carry_rows=32)
    assert native["carry_m"] == 128 and aux["carry_m"] == 32 and aux["carry"].shape == (2, 10, 300)
    sel = oracle.selection_matrix(q[:, 0].float(), k[:, 0].float())
    for rb in range(10):
        want = sel[:, : 32 * rb].sum(dim=1)                 # zero for keys at or after the block, stored or not
        torch.testing.assert_close(aux["carry"][:, rb].cpu(), want, atol=1e-3, rtol=1e-3)
    assert (native["carry"][:, 0] == 0).all() and (aux["carry"][:, 0] == 0).all()


@pytest.mark.parametrize("seq,heads,d", [(300, 3, 64), (1000, 2, 64), (129, 1, 64), (300, 2, 128), (700, 1, 128)])
def test_packed_projection_form_equals_the_plain_call(seq, heads, d):
    """The layout-fused entry (q, k, v read in place from a (B, T, 3, H, D) projection output, merged (B, T, H D)
    output and packed gradients written by the kernels) against the plain call on the three views, and the oracle."""
    g = torch.Generator("cpu").manual_seed(seq)
    b = 2
    qkv = torch.randn(b, seq, 3, heads, d, generator=g).bfloat16().cuda()
    w = torch.randn(b, seq, heads * d, generator=g).bfloat16().cuda()
    assert kernels.packed_supported(qkv)
    x = qkv.clone().requires_grad_(True)
    before = _lib.launch_count()
    y = kernels.selective_attention_packed(x)
    y.backward(w)
    assert _lib.launch_count() - before == 7          # colsum, scan, forward | dbar, backward, 2 x fold: no copy kernels of ours
    torch.cuda.synchronize()
    assert _lib.device_status() == 0
    assert y.shape == (b, seq, heads * d) and y.dtype == torch.bfloat16 and x.grad.shape == qkv.shape

    x2 = qkv.clone().requires_grad_(True)
    q, k, v = (x2[:, :, i].transpose(1, 2) for i in range(3))
    y2 = kernels.selective_attention(q, k, v).to(torch.bfloat16).transpose(1, 2).reshape(b, seq, heads * d)
    y2.backward(w)
    torch.testing.assert_close(y.float(), y2.float(), atol=0, rtol=0)         # the same kernel, the same rounding
    assert _rel(x.grad.float().cpu(), x2.grad.float().cpu()) < 2e-3            # atomics' order only
    qf, kf, vf = (qkv[:, :, i].transpose(1, 2).float().cpu() for i in range(3))
    wf = w.view(b, seq, heads, d).transpose(1, 2).float().cpu()
    want = oracle.attention_grads(qf, kf, vf, wf)
    got = [y.view(b, seq, heads, d).transpose(1, 2).float().cpu()] + [x.grad[:, :, i].transpose(1, 2).float().cpu() for i in range(3)]
    for name, a, bb in zip(("out", "dq", "dk", "dv"), got, want):
        assert _rel(a, bb) < 2e-2, (name, _rel(a, bb))
