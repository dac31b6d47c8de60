"""Generate the golden vectors under tests/golden/ by RUNNING THE REFERENCE ITSELF.

    python tests/golden/make_golden.py --reference <checkout of Selective-Attention-Study>

The reference is a Python package; its paper-listing functions (``selective_logits``,
``selective_attention_reference``) and its attention slot (``mixers.SelectiveAttention`` with
``begin_cache`` / ``step_cache``) run on the CPU.  This script imports them from the checkout,
feeds seeded inputs, differentiates with autograd, and stores inputs and results as small ``.npz``
files.  The tests never need the checkout: they read the files.

Every array is fp32.  File contents:
  q, k, v, d_out          inputs (B, H, T, D)
  out, dq, dk, dv         reference forward and autograd gradients for loss = sum(out * d_out)
  total                   ``selective_logits(...)[1]``  (B, T)   [(B, G, T) for the per-head case]
  exempt, groups          scalars
Decode files add the per-step outputs of the reference's ``step_cache``.
"""

from __future__ import annotations

import argparse
import math
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def _inputs(seed, batch, heads, seq, dim, scale):
    g = torch.Generator("cpu").manual_seed(seed)
    return tuple(scale * torch.randn(batch, heads, seq, dim, generator=g) for _ in range(4))


def _save(name, **arrays):
    out = {}
    for key, val in arrays.items():
        out[key] = val.detach().numpy().astype(np.float32) if torch.is_tensor(val) else np.asarray(val)
    np.savez(os.path.join(HERE, name + ".npz"), **out)
    print(name, {k: v.shape for k, v in out.items()})


def fwd_bwd_case(kernels, name, seed, batch, heads, seq, dim, scale, exempt=1):
    q, k, v, d_out = _inputs(seed, batch, heads, seq, dim, scale)
    qq, kk, vv = (t.clone().requires_grad_(True) for t in (q, k, v))
    out = kernels.selective_attention_reference(qq, kk, vv, exempt=exempt)
    (out * d_out).sum().backward()
    total = kernels.selective_logits(q, k, exempt)[1]
    _save(name, q=q, k=k, v=v, d_out=d_out, out=out, dq=qq.grad, dk=kk.grad, dv=vv.grad, total=total,
          exempt=exempt, groups=1)


def per_head_case(kernels, name, seed, batch, heads, seq, dim, scale):
    """mixers.py:80-84: each head becomes its own one-head sequence."""
    q, k, v, d_out = _inputs(seed, batch, heads, seq, dim, scale)
    qq, kk, vv = (t.clone().requires_grad_(True) for t in (q, k, v))
    flat = lambda t: t.reshape(batch * heads, 1, seq, dim)
    out = kernels.selective_attention_reference(flat(qq), flat(kk), flat(vv)).reshape(batch, heads, seq, dim)
    (out * d_out).sum().backward()
    total = kernels.selective_logits(flat(q), flat(k))[1].reshape(batch, heads, seq)
    _save(name, q=q, k=k, v=v, d_out=d_out, out=out, dq=qq.grad, dk=kk.grad, dv=vv.grad, total=total,
          exempt=1, groups=heads)


def damp_case(kernels, name, seed, heads, seq, dim, scale, train_len):
    """Expected values built the way tests/test_selective_kernels.py:234-241 builds them."""
    q, k, v, _ = _inputs(seed, 1, heads, seq, dim, scale)
    logits, _ = kernels.selective_logits(q, k)
    raw = ((q @ k.transpose(-2, -1)) / math.sqrt(dim)).masked_fill(
        ~torch.ones(seq, seq, dtype=torch.bool).tril(), float("-inf"))
    hist = torch.nan_to_num(raw - logits, nan=0.0)
    factor = (float(train_len) / torch.arange(1, seq + 1, dtype=torch.float32)).clamp(max=1.0)
    _save(name, q=q, k=k, v=v, train_len=train_len,
          out_linear=(raw - hist * factor[:, None]).softmax(-1) @ v,
          out_sqrt=(raw - hist * factor.sqrt()[:, None]).softmax(-1) @ v)


def decode_case(name, attention, seed, heads, d_model, prefill, steps):
    """Drive the reference's own begin_cache / step_cache with identity output projection so the
    per-head attention outputs can be read back."""
    from selective_attention.config import ModelConfig, build_model

    torch.manual_seed(seed)
    cfg = ModelConfig(vocab_size=97, n_layers=1, d_model=d_model, n_heads=heads, context_length=prefill + steps + 4,
                      attention=attention, positional="none")
    attn = build_model(cfg).eval().transformer.h[0].attn
    with torch.no_grad():
        attn.c_proj.weight.copy_(torch.eye(d_model))
        if attn.c_proj.bias is not None:
            attn.c_proj.bias.zero_()
        seq = prefill + steps
        x = torch.randn(2, seq, d_model)
        q, k, v = (t.contiguous() for t in attn._split_heads(x))
        unmerge = lambda y: y.view(2, -1, heads, d_model // heads).transpose(1, 2)
        y0, cache = attn.begin_cache(x[:, :prefill])
        outs = [unmerge(y0)]
        selected_after_prefill = cache["selected"][:, :, :prefill].clone()
        for t in range(prefill, seq):
            outs.append(unmerge(attn.step_cache(x[:, t:t + 1], cache)))
        full, total = attn._attend(q, k, v, want_total=True)
    _save(name, q=q, k=k, v=v, out_steps=torch.cat(outs, dim=2), out_full=full.float(), total_full=total.float(),
          selected_after_prefill=selected_after_prefill, selected_final=cache["selected"][:, :, :seq],
          prefill=prefill, exempt=attn.exempt, groups=attn.groups)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="path of the reference checkout")
    args = ap.parse_args()
    sys.path.insert(0, os.path.join(args.reference, "src"))
    from selective_attention import kernels

    torch.set_num_threads(1)                      # one summation order, whatever the host
    fwd_bwd_case(kernels, "fb_b2_h3_t23_d16", 0, 2, 3, 23, 16, 1.5)
    fwd_bwd_case(kernels, "fb_t1", 1, 2, 2, 1, 16, 1.0)
    fwd_bwd_case(kernels, "fb_t2", 2, 1, 2, 2, 16, 1.0)
    fwd_bwd_case(kernels, "fb_exempt4", 3, 1, 2, 20, 16, 3.0, exempt=4)
    fwd_bwd_case(kernels, "fb_t160_lowscale", 4, 1, 2, 160, 16, 0.3)
    fwd_bwd_case(kernels, "fb_t160_d32", 5, 1, 2, 160, 32, 1.2)
    fwd_bwd_case(kernels, "fb_t130_d64_exempt16", 6, 1, 3, 130, 64, 1.0, exempt=16)
    per_head_case(kernels, "fb_perhead", 7, 2, 4, 30, 16, 1.5)
    damp_case(kernels, "damp_t60", 8, 3, 60, 16, 1.5, train_len=20)
    decode_case("decode_shared", "selective", 9, heads=2, d_model=32, prefill=20, steps=27)
    decode_case("decode_x16", "selective_x16", 10, heads=2, d_model=32, prefill=20, steps=12)
    decode_case("decode_perhead", "selective_perhead", 11, heads=4, d_model=64, prefill=10, steps=10)


if __name__ == "__main__":
    main()
