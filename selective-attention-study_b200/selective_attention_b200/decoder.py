"""Minimal decoder for the full-model benchmark configuration: the harness around the operator, not the
product.  Architecture as the reference's ``DilutionLM`` with Selective Attention in every layer
(``src/selective_attention/model.py:317-418``): pre-LN blocks (``:325-328``), bias-free projections, GELU
MLP of width 4 d (``:276-286``), tied input / output embeddings (``:365-366``), normal(0, 0.02)
initialisation (``:379-385``), no position signal.  The loss is computed over the sequence in chunks so the
(T x vocab) logits never exist at once (the reference does this for evaluation, ``:420-447``).

The attention layer hands the operator the fused QKV projection output as it is (the tensor-core engine
reads strided (B, T, H, D) data through TMA descriptors), gets the merged (B, T, H * D) activation written by
the forward kernel, and gets dq, dk, dv written straight into the projection's gradient: nothing is copied
on either side of the kernels in either pass (bf16; fp32 runs take the unfused call)."""

from __future__ import annotations

import torch
import torch.nn.functional as F
from torch import nn

from . import kernels


class SelectiveSelfAttention(nn.Module):
    def __init__(self, d_model: int, n_heads: int, exempt: int = 1):
        super().__init__()
        self.n_heads, self.d_model, self.exempt = n_heads, d_model, exempt
        self.c_attn = nn.Linear(d_model, 3 * d_model, bias=False)
        self.c_proj = nn.Linear(d_model, d_model, bias=False)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        b, t, _ = x.shape
        qkv = self.c_attn(x).view(b, t, 3, self.n_heads, self.d_model // self.n_heads)
        if kernels.packed_supported(qkv):                                    # bf16: no copy on either side of the kernels
            return self.c_proj(kernels.selective_attention_packed(qkv, exempt=self.exempt))
        q, k, v = (qkv[:, :, i].transpose(1, 2) for i in range(3))          # (B, H, T, D) views, no copy
        y = kernels.selective_attention(q, k, v, exempt=self.exempt).to(x.dtype)
        return self.c_proj(y.transpose(1, 2).reshape(b, t, self.d_model))


class Block(nn.Module):
    def __init__(self, d_model: int, n_heads: int):
        super().__init__()
        self.ln_1 = nn.LayerNorm(d_model, bias=False)
        self.attn = SelectiveSelfAttention(d_model, n_heads)
        self.ln_2 = nn.LayerNorm(d_model, bias=False)
        self.c_fc = nn.Linear(d_model, 4 * d_model, bias=False)
        self.c_proj = nn.Linear(4 * d_model, d_model, bias=False)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        x = x + self.attn(self.ln_1(x))
        return x + self.c_proj(F.gelu(self.c_fc(self.ln_2(x))))


class SelectiveDecoder(nn.Module):
    def __init__(self, vocab_size: int = 50304, n_layers: int = 24, d_model: int = 1024, n_heads: int = 16,
                 loss_chunk: int = 4096):
        super().__init__()
        self.wte = nn.Embedding(vocab_size, d_model)
        self.h = nn.ModuleList([Block(d_model, n_heads) for _ in range(n_layers)])
        self.ln_f = nn.LayerNorm(d_model, bias=False)
        self.loss_chunk = loss_chunk
        for module in self.modules():
            if isinstance(module, (nn.Linear, nn.Embedding)):
                nn.init.normal_(module.weight, mean=0.0, std=0.02)

    def forward(self, idx: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
        x = self.wte(idx)
        for block in self.h:
            x = block(x)
        x = self.ln_f(x)
        total = x.new_zeros((), dtype=torch.float32)
        seq = x.shape[1]
        for a in range(0, seq, self.loss_chunk):                            # tied output embedding, chunked loss
            logits = F.linear(x[:, a:a + self.loss_chunk], self.wte.weight)
            total = total + F.cross_entropy(logits.float().reshape(-1, logits.shape[-1]),
                                            targets[:, a:a + self.loss_chunk].reshape(-1), reduction="sum")
        return total / targets.numel()


def synthetic_batch(batch: int, seq: int, vocab_size: int, bos_id: int, generator: torch.Generator):
    """Uniform random token ids with <BOS> in front: inputs [bos] + w[:-1], targets w (reference data.py:136-139)."""
    w = torch.randint(0, vocab_size, (batch, seq), generator=generator)
    idx = torch.cat([torch.full((batch, 1), bos_id, dtype=w.dtype), w[:, :-1]], dim=1)
    return idx, w
