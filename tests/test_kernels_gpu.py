"""GPU parity tests of the CUDA library against the CPU oracle and the reference-generated golden
vectors.  The cases and tolerances follow the reference's own kernel tests
(tests/test_selective_kernels.py); every call goes through the Python boundary into the C ABI."""

import math

import pytest
import torch

import selective_oracle as oracle
from selective_attention_b200 import kernels

pytestmark = pytest.mark.gpu

FB_CASES = ["fb_b2_h3_t23_d16", "fb_t1", "fb_t2", "fb_exempt4", "fb_t160_lowscale", "fb_t160_d32",
            "fb_t130_d64_exempt16"]


def _qkv(batch, heads, seq, dim, seed=0, scale=1.0, n=3):
    g = torch.Generator("cpu").manual_seed(seed)
    return tuple(scale * torch.randn(batch, heads, seq, dim, generator=g) for _ in range(n))


def _run(q, k, v, d_out, **kw):
    qq, kk, vv = (t.cuda().clone().requires_grad_(True) for t in (q, k, v))
    out = kernels.selective_attention(qq, kk, vv, **kw)
    (out * d_out.cuda()).sum().backward()
    return tuple(t.detach().float().cpu() for t in (out, qq.grad, kk.grad, vv.grad))


def _relerr(got, want):
    return float((got - want).norm() / want.norm().clamp_min(1e-30))


@pytest.mark.parametrize("name", FB_CASES)
def test_golden_forward_backward_ieee(golden, name):
    """fp32 bar: within 1e-4 relative of the reference's own results."""
    g = golden(name)
    got = _run(g["q"], g["k"], g["v"], g["d_out"], dot_precision="ieee", exempt=g["exempt"])
    for key, val in zip(("out", "dq", "dk", "dv"), got):
        torch.testing.assert_close(val, g[key], atol=5e-5, rtol=5e-4, msg=lambda m, key=key: f"{key}: {m}")
        assert _relerr(val, g[key]) < 1e-4 or g[key].norm() == 0, key
    _, aux = kernels.selective_attention_forward(g["q"].cuda(), g["k"].cuda(), g["v"].cuda(), dot_precision="ieee",
                                                 return_aux=True, exempt=g["exempt"])
    torch.testing.assert_close(aux["selected_total"].cpu(), g["total"], atol=2e-4, rtol=2e-5)


def test_golden_per_head_variant(golden):
    g = golden("fb_perhead")
    b, h, t, d = g["q"].shape
    flat = lambda x: x.reshape(b * h, 1, t, d)
    got = _run(flat(g["q"]), flat(g["k"]), flat(g["v"]), flat(g["d_out"]), dot_precision="ieee")
    for key, val in zip(("out", "dq", "dk", "dv"), got):
        torch.testing.assert_close(val.reshape(b, h, t, d), g[key], atol=5e-5, rtol=5e-4)


@pytest.mark.parametrize("seq", [1, 2, 31, 32, 33, 64, 65, 130, 257, 513])
@pytest.mark.parametrize("heads", [1, 3])
def test_forward_matches_oracle(seq, heads):
    q, k, v = _qkv(2, heads, seq, 32, seed=seq, scale=1.5)
    got, aux = kernels.selective_attention_forward(q.cuda(), k.cuda(), v.cuda(), dot_precision="ieee", return_aux=True)
    torch.testing.assert_close(got.cpu(), oracle.attention(q, k, v), atol=2e-5, rtol=2e-5)
    torch.testing.assert_close(aux["selected_total"].cpu(), oracle.selected_total(q, k)[:, 0], atol=2e-4, rtol=2e-5)
    # the saved statistics rebuild the attention: exp2(z - rmax) / rden sums to one over the keys
    z, _ = oracle.history_logits(q, k)
    rebuilt = torch.exp2(z * math.log2(math.e) - aux["rmax"].cpu().view(2, heads, seq, 1)) / aux["rden"].cpu().view(
        2, heads, seq, 1)
    torch.testing.assert_close(rebuilt.sum(-1), torch.ones(2, heads, seq), atol=1e-4, rtol=1e-4)


@pytest.mark.parametrize("dim", [16, 32, 64, 128])
def test_forward_every_head_dim_and_tuning_keywords(dim):
    q, k, v = _qkv(1, 2, 300, dim, seed=dim, scale=1.5)
    for blocks in ((32, 32), (128, 64)):
        got = kernels.selective_attention_forward(q.cuda(), k.cuda(), v.cuda(), dot_precision="ieee",
                                                  block_m=blocks[0], block_n=blocks[1], num_stages=1)
        torch.testing.assert_close(got.cpu(), oracle.attention(q, k, v), atol=2e-5, rtol=2e-5)


@pytest.mark.parametrize("seq", [1, 2, 33, 64, 65, 200, 513])
@pytest.mark.parametrize("heads", [1, 4])
def test_backward_matches_oracle(seq, heads):
    q, k, v, w = _qkv(2, heads, seq, 32, seed=seq + 7, scale=1.5, n=4)
    got = _run(q, k, v, w, dot_precision="ieee")
    want = oracle.attention_grads(q, k, v, w)
    for key, a, b in zip(("out", "dq", "dk", "dv"), got, want):
        torch.testing.assert_close(a, b, atol=5e-5, rtol=5e-4, msg=lambda m, key=key: f"{key}: {m}")


def test_selection_gradient_reaches_head_zero_only_through_the_history_term():
    q, k, v = _qkv(1, 3, 97, 32, seed=3, scale=2.0)
    w = torch.ones(1, 3, 97, 32)
    w[:, 0] = 0                                   # loss on heads >= 1 only
    _, dq, dk, dv = _run(q, k, v, w, dot_precision="ieee")
    _, rq, rk, rv = oracle.attention_grads(q, k, v, w)
    assert rq[:, 0].abs().max() > 1e-4 and dv[:, 0].abs().max() == 0
    for a, b in ((dq, rq), (dk, rk), (dv, rv)):
        torch.testing.assert_close(a, b, atol=5e-5, rtol=5e-4)


def test_long_sequence_low_scale_and_ragged_tail():
    """65 carry rows, a partial last block; low-scale q, k keep F small so far tiles matter."""
    for scale, seed in ((1.2, 5), (0.3, 6)):
        q, k, v, w = _qkv(1, 2, 2049, 32, seed=seed, scale=scale, n=4)
        got = _run(q, k, v, w, dot_precision="ieee")
        want = oracle.attention_grads(q, k, v, w)
        torch.testing.assert_close(got[0], want[0], atol=5e-5, rtol=5e-5)
        for a, b in zip(got[1:], want[1:]):
            assert _relerr(a, b) < 1e-3


@pytest.mark.parametrize("exempt", [1, 3, 16, 40])
def test_exempt_prefix(exempt):
    q, k, v, w = _qkv(2, 4, 257, 32, seed=exempt, scale=1.5, n=4)
    got = _run(q, k, v, w, dot_precision="ieee", exempt=exempt, group=1, bwd_group=1, bwd_block_n=16)
    want = oracle.attention_grads(q, k, v, w, exempt=exempt)
    for key, a, b in zip(("out", "dq", "dk", "dv"), got, want):
        torch.testing.assert_close(a, b, atol=5e-5, rtol=5e-4, msg=lambda m, key=key: f"{key}: {m}")
    _, aux = kernels.selective_attention_forward(q.cuda(), k.cuda(), v.cuda(), dot_precision="ieee", return_aux=True,
                                                 exempt=exempt)
    torch.testing.assert_close(aux["selected_total"].cpu(), oracle.selected_total(q, k, exempt)[:, 0], atol=2e-4,
                               rtol=2e-5)


@pytest.mark.parametrize("damp", ["linear", "sqrt"])
def test_history_damping(golden, damp):
    g = golden("damp_t60")
    q, k, v = (g[n].cuda() for n in "qkv")
    got = kernels.selective_attention_forward(q, k, v, dot_precision="ieee", damp=damp, train_len=g["train_len"])
    torch.testing.assert_close(got.cpu(), g["out_" + damp], atol=2e-5, rtol=2e-5)
    inside = kernels.selective_attention_forward(q, k, v, dot_precision="ieee", damp=damp, train_len=60)
    torch.testing.assert_close(inside, kernels.selective_attention_forward(q, k, v, dot_precision="ieee"))


@pytest.mark.parametrize("precision", ["bf16", "tf32"])
@pytest.mark.parametrize("dim", [64, 128])
def test_low_precision_paths_stay_close(precision, dim):
    """bf16 bar: within 2e-2 (relative norm) on outputs and gradients; gradient dtypes follow inputs."""
    q, k, v = _qkv(2, 4, 400, dim, seed=11)
    if precision == "bf16":
        q, k, v = (t.bfloat16() for t in (q, k, v))
    want = oracle.attention_grads(q.float(), k.float(), v.float(), 2 * oracle.attention(q.float(), k.float(), v.float()))
    qq, kk, vv = (t.cuda().clone().requires_grad_(True) for t in (q, k, v))
    got = kernels.selective_attention(qq, kk, vv, dot_precision=precision)
    assert got.dtype == torch.float32
    assert (got.cpu() - want[0]).abs().max() < 3e-2 and _relerr(got.cpu(), want[0]) < 2e-2
    got.float().pow(2).sum().backward()
    for grad, ref in zip((qq.grad, kk.grad, vv.grad), want[1:]):
        assert grad.dtype == q.dtype
        assert _relerr(grad.float().cpu(), ref) < 2e-2


@pytest.mark.parametrize("dim", [16, 32, 64, 128])
@pytest.mark.parametrize("precision", ["bf16", "tf32", "ieee"])
def test_default_launch_every_head_dim_and_precision(dim, precision):
    q, k, v = _qkv(1, 4, 300, dim, seed=dim)
    if precision == "bf16":
        q, k, v = (t.bfloat16() for t in (q, k, v))
    want = oracle.attention(q, k, v)
    qq, kk, vv = (t.cuda().clone().requires_grad_(True) for t in (q, k, v))
    got = kernels.selective_attention(qq, kk, vv, dot_precision=precision)
    got.float().sum().backward()
    assert (got.cpu() - want).abs().max() < (3e-2 if precision == "bf16" else 5e-5)
    assert all(torch.isfinite(g).all() for g in (qq.grad, kk.grad, vv.grad))


def test_fp16_inputs_and_strided_views():
    """fp16 inputs run the exact path; transposed (B, T, H, D) views are consumed without a copy."""
    q, k, v, w = _qkv(2, 3, 150, 32, seed=21, n=4)
    qh, kh, vh = (t.half() for t in (q, k, v))
    got = _run(qh, kh, vh, w)
    want = oracle.attention_grads(qh.float(), kh.float(), vh.float(), w)
    torch.testing.assert_close(got[0], want[0], atol=5e-5, rtol=5e-4)
    for a, b in zip(got[1:], want[1:]):
        assert _relerr(a, b) < 2e-3                      # gradients are rounded to fp16 on return
    packed = torch.stack([q, k, v], dim=0).permute(0, 1, 3, 2, 4).contiguous().cuda()   # (3, B, T, H, D)
    views = [packed[i].transpose(1, 2) for i in range(3)]
    assert not views[0].is_contiguous()
    out = kernels.selective_attention_forward(*views, dot_precision="ieee")
    torch.testing.assert_close(out.cpu(), oracle.attention(q, k, v), atol=2e-5, rtol=2e-5)


def test_default_precision_follows_the_input_dtype():
    q, k, v = (t.cuda() for t in _qkv(1, 4, 200, 64, seed=8))
    torch.testing.assert_close(kernels.selective_attention_forward(q, k, v),
                               kernels.selective_attention_forward(q, k, v, dot_precision="tf32"))
    qb, kb, vb = q.bfloat16(), k.bfloat16(), v.bfloat16()
    torch.testing.assert_close(kernels.selective_attention_forward(qb, kb, vb),
                               kernels.selective_attention_forward(qb, kb, vb, dot_precision="bf16"))


def test_bad_inputs_raise_clear_errors():
    q, k, v = (t.cuda() for t in _qkv(1, 2, 64, 32))
    with pytest.raises(ValueError, match="must all be"):
        kernels.selective_attention(q, k[:, :, :32], v)
    with pytest.raises(ValueError, match="CUDA"):
        kernels.selective_attention(q.cpu(), k.cpu(), v.cpu())
    with pytest.raises(ValueError, match="dtype"):
        kernels.selective_attention(q.double(), k.double(), v.double())
    with pytest.raises(ValueError, match="head_dim"):
        kernels.selective_attention(q[..., :24], k[..., :24], v[..., :24])
    with pytest.raises(ValueError, match="dot_precision"):
        kernels.selective_attention(q, k, v, dot_precision="fp8")
    with pytest.raises(ValueError, match="exempt"):
        kernels.selective_attention(q, k, v, exempt=0)
    with pytest.raises(ValueError, match="bwd_group"):
        kernels.selective_attention(q.clone().requires_grad_(True), k, v, bwd_group=4).sum().backward()
    with pytest.raises(ValueError, match="damp"):
        kernels.selective_attention_forward(q, k, v, damp="cubic", train_len=10)
    with pytest.raises(ValueError, match="train_len"):
        kernels.selective_attention_forward(q, k, v, damp="linear")
    with pytest.raises(ValueError, match="multiples of 32"):
        kernels.selective_attention_forward(q, k, v, block_n=48)
    with pytest.raises(TypeError):
        kernels.selective_attention_forward(q, k, v, None, None, 32, False, 4, None, None, 1, "linear")
    assert kernels.supported(q) and not kernels.supported(q.cpu()) and not kernels.supported(q[..., :24])
