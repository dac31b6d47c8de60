"""The full-model harness (bench.py --workload c5): a small decoder through the operator equals the same
decoder through the dense listing, loss and every parameter gradient (the reference checks the same for its
model, tests/test_selective_model.py:56-71), and a bf16 autocast step is finite."""

import pytest
import torch

from selective_attention_b200 import decoder, kernels

pytestmark = pytest.mark.gpu


def _loss_and_grads(model, idx, tgt, dense: bool, autocast: bool):
    original = kernels.selective_attention
    if dense:
        decoder.kernels.selective_attention = lambda q, k, v, exempt=1: kernels.selective_attention_reference(q, k, v, exempt)
    try:
        model.zero_grad()
        with torch.autocast("cuda", dtype=torch.bfloat16, enabled=autocast):
            loss = model(idx, tgt)
        loss.backward()
        return loss.detach(), torch.cat([p.grad.flatten().float() for p in model.parameters()])
    finally:
        decoder.kernels.selective_attention = original


def test_decoder_through_the_operator_matches_the_dense_listing():
    torch.manual_seed(1)
    model = decoder.SelectiveDecoder(vocab_size=97, n_layers=3, d_model=128, n_heads=2, loss_chunk=128).cuda()
    gen = torch.Generator("cpu").manual_seed(2)
    idx, tgt = (t.cuda() for t in decoder.synthetic_batch(2, 300, 97, 96, gen))
    assert (idx[:, 0] == 96).all() and torch.equal(idx[:, 1:], tgt[:, :-1])
    loss_a, grad_a = _loss_and_grads(model, idx, tgt, dense=False, autocast=False)      # fp32: exact engine
    loss_b, grad_b = _loss_and_grads(model, idx, tgt, dense=True, autocast=False)
    torch.testing.assert_close(loss_a, loss_b, atol=1e-5, rtol=1e-5)
    assert (grad_a - grad_b).norm() / grad_b.norm() < 2e-3
    loss_c, grad_c = _loss_and_grads(model, idx, tgt, dense=False, autocast=True)       # bf16: tensor-core engine
    assert torch.isfinite(loss_c) and torch.isfinite(grad_c).all()
    assert abs(float(loss_c) - float(loss_b)) < 2e-2
    assert (grad_c - grad_b).norm() / grad_b.norm() < 5e-2
