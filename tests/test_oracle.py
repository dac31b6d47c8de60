"""The CPU oracle against the golden vectors the reference itself produced (tests/golden)."""

import pytest
import torch

import selective_oracle as oracle

FB_CASES = ["fb_b2_h3_t23_d16", "fb_t1", "fb_t2", "fb_exempt4", "fb_t160_lowscale", "fb_t160_d32",
            "fb_t130_d64_exempt16", "fb_perhead"]


@pytest.mark.parametrize("name", FB_CASES)
def test_forward_and_closed_form_gradients_match_the_reference(golden, name):
    g = golden(name)
    out, dq, dk, dv = oracle.attention_grads(g["q"], g["k"], g["v"], g["d_out"], g["exempt"], g["groups"])
    for key, got in (("out", out), ("dq", dq), ("dk", dk), ("dv", dv)):
        torch.testing.assert_close(got, g[key], atol=3e-5, rtol=1e-4, msg=lambda m, key=key: f"{key}: {m}")
    total = oracle.selected_total(g["q"], g["k"], g["exempt"], g["groups"])
    want = g["total"] if g["total"].dim() == 3 else g["total"][:, None]
    torch.testing.assert_close(total, want, atol=1e-4, rtol=1e-5)
    torch.testing.assert_close(oracle.attention(g["q"], g["k"], g["v"], g["exempt"], g["groups"]), g["out"],
                               atol=1e-5, rtol=1e-5)


def test_fp64_oracle_agrees_with_fp32_reference(golden):
    g = golden("fb_t160_d32")
    out, dq, dk, dv = oracle.attention_grads(g["q"], g["k"], g["v"], g["d_out"], dtype=torch.float64)
    for key, got in (("out", out), ("dq", dq), ("dk", dk), ("dv", dv)):
        assert (got.float() - g[key]).norm() / g[key].norm() < 1e-5, key


def test_per_query_loop_is_the_same_function(golden):
    g = golden("fb_b2_h3_t23_d16")
    torch.testing.assert_close(oracle.per_query_loop(g["q"], g["k"], g["v"]), g["out"], atol=1e-5, rtol=1e-5)
    g = golden("fb_exempt4")
    torch.testing.assert_close(oracle.per_query_loop(g["q"], g["k"], g["v"], 4), g["out"], atol=1e-5, rtol=1e-5)


def test_mask_rules(golden):
    """BOS column and diagonal are never reduced; first and last totals are zero
    (reference tests/test_selective_kernels.py:43-49,193-200)."""
    g = golden("fb_exempt4")
    z, total = oracle.history_logits(g["q"], g["k"], 4)
    raw = (g["q"] @ g["k"].transpose(-2, -1)) / 4.0
    causal = torch.ones(20, 20, dtype=torch.bool).tril()
    torch.testing.assert_close(z[..., :4], raw.masked_fill(~causal, float("-inf"))[..., :4])
    torch.testing.assert_close(z.diagonal(dim1=-2, dim2=-1), raw.diagonal(dim1=-2, dim2=-1))
    assert torch.all(total[..., :4] == 0) and total[0, -1] == 0 and float(total.sum()) > 0
    with pytest.raises(ValueError, match="exempt"):
        oracle.attention(g["q"], g["k"], g["v"], exempt=0)


def test_damped_forward(golden):
    g = golden("damp_t60")
    for mode in ("linear", "sqrt"):
        got = oracle.damped_attention(g["q"], g["k"], g["v"], mode, g["train_len"])
        torch.testing.assert_close(got, g["out_" + mode], atol=1e-5, rtol=1e-5)
    inside = oracle.damped_attention(g["q"], g["k"], g["v"], "linear", 60)
    torch.testing.assert_close(inside, oracle.attention(g["q"], g["k"], g["v"]), atol=1e-6, rtol=1e-6)


def test_tail_rows_and_chunked_sequence_match_the_dense_form(golden):
    g = golden("fb_t160_d32")
    rows, out, total = oracle.tail_rows(g["q"], g["k"], g["v"], tail=37, chunk=50)
    torch.testing.assert_close(out, g["out"][:, :, rows], atol=1e-5, rtol=1e-5)
    torch.testing.assert_close(total, g["total"], atol=1e-4, rtol=1e-5)
    out, dq, dk, dv, total = oracle.sequence_fwd_bwd(g["q"][0], g["k"][0], g["v"][0], g["d_out"][0], head_chunk=1)
    for key, got in (("out", out), ("dq", dq), ("dk", dk), ("dv", dv)):
        torch.testing.assert_close(got, g[key][0], atol=3e-5, rtol=1e-4, msg=lambda m, key=key: f"{key}: {m}")
    torch.testing.assert_close(total, g["total"][0], atol=1e-4, rtol=1e-5)


@pytest.mark.parametrize("name", ["decode_shared", "decode_x16", "decode_perhead"])
def test_decode_steps_match_the_reference_cache_path(golden, name):
    g = golden(name)
    q, k, v = g["q"], g["k"], g["v"]
    b, h, seq, d = q.shape
    p, groups, exempt = g["prefill"], g["groups"], g["exempt"]
    cache = {"k": torch.zeros(b, h, seq + 2, d), "v": torch.zeros(b, h, seq + 2, d), "len": p,
             "selected": torch.zeros(b, groups, seq + 2)}
    cache["k"][:, :, :p], cache["v"][:, :, :p] = k[:, :, :p], v[:, :, :p]
    cache["selected"][:, :, :p] = oracle.selected_total(q[:, :, :p], k[:, :, :p], exempt, groups)
    torch.testing.assert_close(cache["selected"][:, :, :p], g["selected_after_prefill"], atol=1e-5, rtol=1e-5)
    torch.testing.assert_close(oracle.attention(q[:, :, :p], k[:, :, :p], v[:, :, :p], exempt, groups),
                               g["out_steps"][:, :, :p], atol=1e-5, rtol=1e-5)
    for t in range(p, seq):
        y = oracle.decode_step(cache, q[:, :, t:t + 1], k[:, :, t:t + 1], v[:, :, t:t + 1], exempt, groups)
        torch.testing.assert_close(y, g["out_steps"][:, :, t:t + 1], atol=1e-5, rtol=1e-5)
        torch.testing.assert_close(y, g["out_full"][:, :, t:t + 1], atol=2e-5, rtol=2e-5)
    torch.testing.assert_close(cache["selected"][:, :, :seq], g["selected_final"], atol=1e-5, rtol=1e-5)
    with pytest.raises(ValueError, match="capacity"):
        cache["len"] = seq + 2
        oracle.decode_step(cache, q[:, :, :1], k[:, :, :1], v[:, :, :1], exempt, groups)
