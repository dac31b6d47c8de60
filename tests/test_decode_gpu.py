"""Cached prefill + decode on the device against the reference-generated golden steps and the oracle."""

import pytest
import torch

import selective_oracle as oracle
from selective_attention_b200 import mixers

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
