"""CPU oracle for the Selective Attention operator.  TEST INFRASTRUCTURE ONLY.

This file restates, in plain dense torch on the CPU, the algorithm of the reference's operator
path.  It is the checker the parity tests, the smoke run and the benchmark's CPU-baseline leg use;
the product path (the CUDA library and its host wrapper) never imports it.

Parity pin: every function below is checked in ``tests/test_oracle.py`` against golden vectors that
``tests/golden/make_golden.py`` produced by importing and running the reference's own
``selective_attention.kernels`` / ``selective_attention.mixers`` code.

What each function follows (paths inside the reference project):

=========================  ==========================================================================
``history_logits``         ``src/selective_attention/kernels.py:61-76``  (``selective_logits``)
``attention``              ``src/selective_attention/kernels.py:79-83``  (``selective_attention_reference``)
``per_query_loop``         ``tests/test_selective_kernels.py:24-40``     (the definition, one query at a time)
``attention_grads``        ``src/selective_attention/kernels.py:204-268, 621-666`` (the backward's algebra,
                           written densely: dV, dz, dK, dQ, the suffix sum U, the gated head-0 gradient)
``damped_attention``       ``src/selective_attention/kernels.py:179-182`` (evaluation-only damping of F)
``window_rows``            ``tests/test_selective_kernels.py:310-330``   (a window of query rows of a long
``tail_rows``              sequence: the selection of earlier queries summed in chunks; the tail is the
                           reference's own form, the window generalises its start)
``decode_step``            ``src/selective_attention/mixers.py:115-130`` (one cached decode step)
``sequence_fwd_bwd``       the same algebra as ``attention`` / ``attention_grads`` for one sequence at a
                           length where (H, T, T) does not fit: F is built once, heads go in chunks
=========================  ==========================================================================

Shapes: q, k, v, d_out are (B, H, T, D); ``groups`` selectors per sequence means heads are split in
``groups`` contiguous runs and the first head of each run supplies the selection
(``mixers.py:66,80-84``); ``groups=1`` is the paper's operator (head 0 selects for all heads).
"""

from __future__ import annotations

import math

import torch


def _check_exempt(exempt: int) -> int:
    if int(exempt) != exempt or exempt < 1:
        raise ValueError(f"exempt must be an integer >= 1; got {exempt}")
    return int(exempt)


def _selector_view(t: torch.Tensor, groups: int) -> torch.Tensor:
    """(B, H, T, D) -> (B * groups, H / groups, T, D): each selector group becomes a sequence."""
    b, h, s, d = t.shape
    if h % groups:
        raise ValueError("heads must divide into selector groups")
    return t.reshape(b * groups, h // groups, s, d)


def selection_matrix(q0: torch.Tensor, k0: torch.Tensor, exempt: int = 1) -> torch.Tensor:
    """S[r, j] = relu(q0[r].k0[j] / sqrt(D)) for exempt <= j < r, else 0.   q0, k0: (..., T, D)."""
    exempt = _check_exempt(exempt)
    seq, dim = q0.shape[-2], q0.shape[-1]
    l0 = (q0 @ k0.transpose(-2, -1)) / math.sqrt(dim)
    rows = torch.arange(seq, device=q0.device)[:, None]
    cols = torch.arange(seq, device=q0.device)[None, :]
    allowed = (cols < rows) & (cols >= exempt)
    return torch.where(allowed & (l0 > 0), l0, torch.zeros((), dtype=l0.dtype, device=q0.device))


def history_logits(q: torch.Tensor, k: torch.Tensor, exempt: int = 1, dtype=torch.float32):
    """(L - F) with -inf above the diagonal, (B, H, T, T), and the per-key totals (B, T)."""
    q, k = q.to(dtype), k.to(dtype)
    seq, dim = q.shape[-2], q.shape[-1]
    logits = (q @ k.transpose(-2, -1)) / math.sqrt(dim)
    upper = torch.ones(seq, seq, dtype=torch.bool).triu(1)
    logits = logits.masked_fill(upper, float("-inf"))
    sel = selection_matrix(q[:, 0], k[:, 0], exempt)                 # (B, T, T)
    total = sel.sum(dim=-2)
    history = torch.cumsum(sel, dim=-2) - sel                        # exclusive: queries r < i
    return logits - history[:, None], total


def attention(q, k, v, exempt: int = 1, groups: int = 1, dtype=torch.float32) -> torch.Tensor:
    """out = softmax(L - F) @ v in ``dtype`` (fp32 like the reference; fp64 for tight checks)."""
    shape = q.shape
    q, k, v = (_selector_view(t, groups) for t in (q, k, v))
    z, _ = history_logits(q, k, exempt, dtype)
    return (z.softmax(dim=-1) @ v.to(dtype)).reshape(shape)


def selected_total(q, k, exempt: int = 1, groups: int = 1, dtype=torch.float32) -> torch.Tensor:
    """(B, groups, T): selection every key received from all T queries (the decode accumulator)."""
    b, _, s, _ = q.shape
    qs, ks = _selector_view(q, groups), _selector_view(k, groups)
    return selection_matrix(qs[:, 0].to(dtype), ks[:, 0].to(dtype), exempt).sum(dim=-2).reshape(b, groups, s)


def per_query_loop(q, k, v, exempt: int = 1) -> torch.Tensor:
    """The definition one query at a time (small cases only)."""
    b, h, seq, dim = q.shape
    out = torch.zeros(b, h, seq, dim, dtype=torch.float32)
    for bi in range(b):
        received = torch.zeros(seq)
        for i in range(seq):
            logit = torch.einsum("hd,hjd->hj", q[bi, :, i].float(), k[bi, :, : i + 1].float()) / dim ** 0.5
            prob = (logit - received[: i + 1]).softmax(-1)
            out[bi, :, i] = torch.einsum("hj,hjd->hd", prob, v[bi, :, : i + 1].float())
            mine = torch.relu(logit[0]).clone()
            mine[:exempt] = 0.0
            mine[i] = 0.0
            received[: i + 1] += mine
    return out


def attention_grads(q, k, v, d_out, exempt: int = 1, groups: int = 1, dtype=torch.float32):
    """(out, dq, dk, dv) from the backward's closed form; no autograd.

    A = softmax(z);  dbar_i = dO_i . out_i;  dV = A^T dO;  dz = A * (dO V^T - dbar)
    dK = s dz^T Q;  dQ = s dz K;  U[r, j] = sum_h sum_{i > r} dz_h[i, j];  g = gate ? -U : 0
    dK_0 += s g^T Q_0;  dQ_0 += s g K_0            (head 0 of each selector group)
    """
    shape = q.shape
    q, k, v, d_out = (_selector_view(t, groups).to(dtype) for t in (q, k, v, d_out))
    seq, dim = q.shape[-2], q.shape[-1]
    s = 1.0 / math.sqrt(dim)
    z, _ = history_logits(q, k, exempt, dtype)
    prob = z.softmax(dim=-1)
    out = prob @ v
    dbar = (d_out * out).sum(dim=-1, keepdim=True)
    dv = prob.transpose(-2, -1) @ d_out
    dz = prob * (d_out @ v.transpose(-2, -1) - dbar)
    dk = s * (dz.transpose(-2, -1) @ q)
    dq = s * (dz @ k)
    dz_all = dz.sum(dim=1)                                            # (Bsel, T, T): all heads of the group
    # suffix over strictly later queries: U[r] = sum_{i > r} dz[i]
    later = torch.flip(torch.cumsum(torch.flip(dz_all, [-2]), dim=-2), [-2]) - dz_all
    gate = selection_matrix(q[:, 0], k[:, 0], exempt) > 0
    g = torch.where(gate, -later, torch.zeros((), dtype=dtype))
    dk[:, 0] += s * (g.transpose(-2, -1) @ q[:, 0])
    dq[:, 0] += s * (g @ k[:, 0])
    return tuple(t.reshape(shape) for t in (out, dq, dk, dv))


def damped_attention(q, k, v, damp: str, train_len: int, exempt: int = 1, dtype=torch.float32):
    """Forward with F scaled per query row by min(1, train_len/(i+1)) ('linear') or its sqrt."""
    q, k, v = q.to(dtype), k.to(dtype), v.to(dtype)
    seq, dim = q.shape[-2], q.shape[-1]
    raw = (q @ k.transpose(-2, -1)) / math.sqrt(dim)
    sel = selection_matrix(q[:, 0], k[:, 0], exempt)
    history = torch.cumsum(sel, dim=-2) - sel
    factor = (float(train_len) / torch.arange(1, seq + 1, dtype=dtype)).clamp(max=1.0)
    if damp == "sqrt":
        factor = factor.sqrt()
    elif damp != "linear":
        raise ValueError("damp must be 'linear' or 'sqrt'")
    z = raw - (history * factor[:, None])[:, None]
    z = z.masked_fill(torch.ones(seq, seq, dtype=torch.bool).triu(1), float("-inf"))
    return z.softmax(dim=-1) @ v


def window_rows(q, k, v, start: int, stop: int, exempt: int = 1, chunk: int = 1024, dtype=torch.float32):
    """Outputs of the queries [start, stop) and the selection every key has received from the queries
    before ``stop``, without a (T, T) tensor: the selection of the earlier queries is summed in chunks.
    Runs where its inputs live (dense torch ops either way)."""
    b, h, seq, dim = q.shape
    s = 1.0 / math.sqrt(dim)
    dev = q.device
    keys = torch.arange(stop, device=dev)
    q0, k0 = q[:, 0].to(dtype), k[:, 0, :stop].to(dtype)

    def sel(rows):
        l0 = (q0[:, rows] @ k0.transpose(-2, -1)) * s
        ok = (keys[None, :] < rows[:, None]) & (keys >= exempt)[None, :]
        return torch.relu(l0) * ok

    earlier = torch.zeros(b, stop, dtype=dtype, device=dev)
    for a in range(0, start, chunk):
        earlier += sel(torch.arange(a, min(a + chunk, start), device=dev)).sum(dim=1)
    rows = torch.arange(start, stop, device=dev)
    st = sel(rows)
    history = earlier[:, None, :] + torch.cumsum(st, dim=1) - st
    z = (q[:, :, rows].to(dtype) @ k[:, :, :stop].to(dtype).transpose(-2, -1)) * s - history[:, None]
    z = z.masked_fill(keys[None, None, None, :] > rows[None, None, :, None], float("-inf"))
    return rows, z.softmax(dim=-1) @ v[:, :, :stop].to(dtype), earlier + st.sum(dim=1)


def tail_rows(q, k, v, tail: int, exempt: int = 1, chunk: int = 1024, dtype=torch.float32):
    """Outputs of the last ``tail`` queries and the per-key totals, without a (T, T) tensor."""
    seq = q.shape[2]
    return window_rows(q, k, v, seq - tail, seq, exempt, chunk, dtype)


def sequence_fwd_bwd(q, k, v, d_out, exempt: int = 1, head_chunk: int = 2, dtype=torch.float32):
    """(out, dq, dk, dv, total) for ONE sequence (H, T, D) with F (T, T) built once and the heads
    processed ``head_chunk`` at a time, so peak memory is (head_chunk + 3) * T * T values.  Runs where its
    inputs live."""
    h, seq, dim = q.shape
    dev = q.device
    s = 1.0 / math.sqrt(dim)
    q, k, v, d_out = (t.to(dtype) for t in (q, k, v, d_out))
    sel = selection_matrix(q[0], k[0], exempt)
    gate = sel > 0
    total = sel.sum(dim=0)
    history = torch.cumsum(sel, dim=0) - sel
    del sel
    upper = torch.ones(seq, seq, dtype=torch.bool, device=dev).triu(1)
    out = torch.empty_like(q)
    dq, dk, dv = torch.empty_like(q), torch.empty_like(q), torch.empty_like(q)
    dz_all = torch.zeros(seq, seq, dtype=dtype, device=dev)
    for a in range(0, h, head_chunk):
        hs = slice(a, min(a + head_chunk, h))
        z = (q[hs] @ k[hs].transpose(-2, -1)) * s - history
        prob = z.masked_fill(upper, float("-inf")).softmax(dim=-1)
        del z
        out[hs] = prob @ v[hs]
        dbar = (d_out[hs] * out[hs]).sum(dim=-1, keepdim=True)
        dv[hs] = prob.transpose(-2, -1) @ d_out[hs]
        dz = prob * (d_out[hs] @ v[hs].transpose(-2, -1) - dbar)
        del prob
        dk[hs] = s * (dz.transpose(-2, -1) @ q[hs])
        dq[hs] = s * (dz @ k[hs])
        dz_all += dz.sum(dim=0)
        del dz
    later = torch.flip(torch.cumsum(torch.flip(dz_all, [0]), dim=0), [0]) - dz_all
    del dz_all
    g = torch.where(gate, -later, torch.zeros((), dtype=dtype, device=dev))
    del later
    dk[0] += s * (g.t() @ q[0])
    dq[0] += s * (g @ k[0])
    return out, dq, dk, dv, total


def decode_step(cache: dict, q1, k1, v1, exempt: int = 1, groups: int = 1):
    """One cached decode step.  cache = {"k","v": (B,H,cap,D), "len": int, "selected": (B,G,cap) fp32};
    q1, k1, v1: (B, H, 1, D).  Appends k1/v1, returns y (B, H, 1, D) fp32, updates ``selected`` in place
    AFTER the output was formed (the new query's own selection; positions < exempt and self are zero)."""
    t = cache["len"]
    if t >= cache["k"].shape[2]:
        raise ValueError("decode step past the cache capacity")
    cache["k"][:, :, t] = k1[:, :, 0]
    cache["v"][:, :, t] = v1[:, :, 0]
    cache["len"] = t = t + 1
    kk, vv = cache["k"][:, :, :t].float(), cache["v"][:, :, :t].float()
    heads, dim = q1.shape[1], q1.shape[-1]
    per = heads // groups
    raw = (q1.float() @ kk.transpose(-2, -1)) / math.sqrt(dim)              # (B, H, 1, t)
    received = cache["selected"][:, :, :t]
    y = (raw - received.repeat_interleave(per, dim=1)[:, :, None, :]).softmax(dim=-1) @ vv
    mine = torch.relu(raw[:, ::per, 0]).clone()
    mine[..., :exempt] = 0.0
    mine[..., t - 1] = 0.0
    received += mine
    return y
