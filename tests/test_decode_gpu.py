"""Cached prefill + decode on the device against the reference-generated golden steps and the oracle."""

import pytest
import torch

import selective_oracle as oracle
from selective_attention_b200 import _lib, mixers

pytestmark = pytest.mark.gpu

VARIANT = {"decode_shared": "selective", "decode_x16": "selective_x16", "decode_perhead": "selective_perhead"}


@pytest.mark.parametrize("name", list(VARIANT))
def test_prefill_then_decode_matches_the_reference_steps(golden, name):
    g = golden(name)
    q, k, v = (g[n].cuda() for n in "qkv")
    b, h, seq, d = q.shape
    p = g["prefill"]
    slot = mixers.SelectiveAttentionSlot.from_variant(VARIANT[name], n_heads=h, context_length=seq + 3)
    slot.dot_precision = "ieee"
    assert slot.groups == g["groups"] and slot.exempt == g["exempt"]
    with torch.no_grad():
        y, cache = slot.begin_cache(q[:, :, :p], k[:, :, :p], v[:, :, :p])
    torch.testing.assert_close(y.cpu(), g["out_steps"][:, :, :p], atol=2e-5, rtol=2e-5)
    torch.testing.assert_close(cache["selected"][:, :, :p].cpu(), g["selected_after_prefill"], atol=2e-5, rtol=2e-5)
    for t in range(p, seq):
        y = slot.step_cache(q[:, :, t:t + 1], k[:, :, t:t + 1], v[:, :, t:t + 1], cache)
        torch.testing.assert_close(y.cpu(), g["out_steps"][:, :, t:t + 1], atol=2e-5, rtol=2e-5)
    assert cache["len"] == seq
    torch.testing.assert_close(cache["selected"][:, :, :seq].cpu(), g["selected_final"], atol=5e-5, rtol=5e-5)
    torch.testing.assert_close(cache["k"][:, :, :seq].cpu(), g["k"])
    cache["len"] = cache["k"].shape[2]
    with pytest.raises(ValueError, match="capacity"):
        slot.step_cache(q[:, :, :1], k[:, :, :1], v[:, :, :1], cache)


@pytest.mark.parametrize("dtype,dim", [(torch.bfloat16, 64), (torch.float16, 128), (torch.float32, 16)])
def test_decode_over_several_splits(dtype, dim):
    """A cache longer than one 512-key split, every cache dtype."""
    gen = torch.Generator("cpu").manual_seed(dim)
    b, h, t0, steps = 2, 4, 1200, 3
    q, k, v = (torch.randn(b, h, t0 + steps, dim, generator=gen).to(dtype) for _ in range(3))
    q = q * 0.5
    ref = {"k": torch.zeros(b, h, t0 + steps, dim, dtype=dtype), "v": torch.zeros(b, h, t0 + steps, dim, dtype=dtype),
           "len": t0, "selected": torch.zeros(b, 2, t0 + steps)}
    ref["k"][:, :, :t0], ref["v"][:, :, :t0] = k[:, :, :t0], v[:, :, :t0]
    ref["selected"][:, :, :t0] = torch.rand(b, 2, t0, generator=gen) * 3
    dev = {key: (val.cuda() if torch.is_tensor(val) else val) for key, val in ref.items()}
    slot = mixers.SelectiveAttentionSlot(n_heads=h, context_length=t0 + steps)
    for t in range(t0, t0 + steps):
        want = oracle.decode_step(ref, q[:, :, t:t + 1], k[:, :, t:t + 1], v[:, :, t:t + 1], groups=2)
        got = slot.step_cache(q[:, :, t:t + 1].cuda(), k[:, :, t:t + 1].cuda(), v[:, :, t:t + 1].cuda(), dev)
        assert got.dtype == dtype
        tol = 2e-5 if dtype == torch.float32 else 2e-2
        torch.testing.assert_close(got.float().cpu(), want, atol=tol, rtol=tol)
    torch.testing.assert_close(dev["selected"].cpu(), ref["selected"], atol=1e-4, rtol=1e-4)


@pytest.mark.parametrize("first,second,heads,per_head", [(256, 200, 3, False), (300, 333, 2, False), (130, 127, 2, True),
                                                         (1000, 1049, 4, False)])
def test_chunked_prefill_equals_one_prefill_and_then_decodes(first, second, heads, per_head):
    """begin_cache on the first chunk + extend_cache on the second must give the rows and the per-key selection of a
    single prefill over all tokens (cached length aligned to the 128-row tiles or not), and the cache must then decode
    like the oracle's."""
    from selective_attention_b200 import mixers
    g = torch.Generator("cpu").manual_seed(first + second)
    total = first + second
    q, k, v = (torch.randn(2, heads, total + 1, 64, generator=g).bfloat16().cuda() for _ in range(3))
    slot = mixers.SelectiveAttentionSlot(n_heads=heads, context_length=total + 8, per_head=per_head)
    whole, whole_total = slot.attend(q[:, :, :total], k[:, :, :total], v[:, :, :total], want_total=True)
    y1, cache = slot.begin_cache(q[:, :, :first], k[:, :, :first], v[:, :, :first])
    y2 = slot.extend_cache(q[:, :, first:total], k[:, :, first:total], v[:, :, first:total], cache)
    torch.cuda.synchronize()
    assert _lib.device_status() == 0 and cache["len"] == total
    torch.testing.assert_close(y1.float(), whole[:, :, :first].float(), atol=0, rtol=0)
    torch.testing.assert_close(y2.float(), whole[:, :, first:].float(), atol=2e-2, rtol=2e-2)
    assert float((y2.float() - whole[:, :, first:].float()).norm() / whole[:, :, first:].float().norm()) < 2e-3
    torch.testing.assert_close(cache["selected"][:, :, :total], whole_total, atol=1e-3, rtol=1e-4)
    assert (cache["selected"][:, :, total:] == 0).all()
    # one decode step on the extended cache against the oracle's step on a float copy of it
    groups = heads if per_head else 1
    ref = {"k": cache["k"].float().cpu().clone(), "v": cache["v"].float().cpu().clone(), "len": total,
           "selected": cache["selected"].cpu().clone()}
    want = oracle.decode_step(ref, q[:, :, total:].float().cpu(), k[:, :, total:].float().cpu(), v[:, :, total:].float().cpu(),
                              groups=groups)
    got = slot.step_cache(q[:, :, total:], k[:, :, total:], v[:, :, total:], cache)
    torch.testing.assert_close(got.float().cpu(), want, atol=2e-2, rtol=2e-2)
    torch.testing.assert_close(cache["selected"].cpu(), ref["selected"], atol=2e-3, rtol=1e-3)
