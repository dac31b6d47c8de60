"""The attention-slot logic of the reference's ``mixers.SelectiveAttention`` at the q / k / v level.

The reference's layer (``src/selective_attention/mixers.py:50-130``) owns the projections and delegates
the attention itself to three methods; this class is those three methods without the projections, so
the reference's layer can call it after ``_split_heads`` and before ``_merge_heads``:

    _attend      -> attend(q, k, v, want_total)            (reference :76-98)
    begin_cache  -> begin_cache(q, k, v, capacity)         (reference :105-113 with model.py:76-83)
    (none)       -> extend_cache(q, k, v, cache)           a further prompt chunk; the reference prefills once
    step_cache   -> step_cache(q1, k1, v1, cache)          (reference :115-130 with model.py:86-93)

Variants as in the reference (:16-22): "selective" (head 0 selects, <BOS> exempt), "selective_x16"
(first 16 positions exempt), "selective_perhead" (every head is its own selector).
"""

from __future__ import annotations

import torch

from . import kernels

VARIANTS = {"selective": (1, False), "selective_x16": (16, False), "selective_perhead": (1, True)}
MIXER_TYPES = tuple(VARIANTS)


class SelectiveAttentionSlot:
    def __init__(self, n_heads: int, context_length: int, exempt: int = 1, per_head: bool = False,
                 dropout: float = 0.0):
        self.n_heads = int(n_heads)
        self.context_length = int(context_length)
        self.exempt = kernels._check_exempt(exempt)
        self.groups = self.n_heads if per_head else 1
        self.dropout = float(dropout)
        self.training = False
        self.use_kernel = True
        self.history_damp = "none"      # evaluation only; forward / prefill
        self.dot_precision = None       # None: "bf16" for bf16 inputs, else "tf32"

    @classmethod
    def from_variant(cls, name: str, n_heads: int, context_length: int, **kw):
        exempt, per_head = VARIANTS[name]
        return cls(n_heads, context_length, exempt=exempt, per_head=per_head, **kw)

    def _kernel_ok(self, q: torch.Tensor) -> bool:
        return self.use_kernel and kernels.supported(q) and (not self.training or self.dropout == 0.0)

    def attend(self, q, k, v, want_total: bool = False):
        """(B, H, T, D) outputs in v's dtype and, on request, the (B, G, T) selection totals."""
        b, h, t, d = q.shape
        g = self.groups
        if g > 1:                       # every selector group becomes its own sequence
            q, k, v = (x.reshape(b * g, h // g, t, d) for x in (q, k, v))
        y, total = self._attend_shared(q, k, v, want_total)
        return y.reshape(b, h, t, d), (None if total is None else total.reshape(b, g, t))

    def _attend_shared(self, q, k, v, want_total: bool):
        if self._kernel_ok(q):
            if want_total or not torch.is_grad_enabled():
                y, aux = kernels.selective_attention_forward(
                    q, k, v, dot_precision=self.dot_precision, return_aux=True, exempt=self.exempt,
                    damp=self.history_damp, train_len=self.context_length)
                return y.to(v.dtype), aux["selected_total"]
            y = kernels.selective_attention(q, k, v, dot_precision=self.dot_precision, exempt=self.exempt)
            return y.to(v.dtype), None
        # off-kernel path: the dense listing, exactly as the reference falls back (CPU tensors, dropout)
        with torch.autocast(q.device.type, enabled=False):
            logits, total = kernels.selective_logits(q, k, self.exempt)
            return (logits.softmax(dim=-1) @ v.float()).to(v.dtype), total

    def begin_cache(self, q, k, v, capacity: int | None = None, live_keys: bool = False):
        """Prefill: outputs plus the decode cache {"k", "v", "len", "selected"}.  ``live_keys`` adds ``"key_norms"``,
        with which the decode steps leave out the part of the cache that no longer carries weight."""
        b, h, t, d = k.shape
        y, total = self.attend(q, k, v, want_total=True)
        capacity = max(capacity if capacity is not None else self.context_length, t)
        cache = {"k": k.new_zeros(b, h, capacity, d), "v": v.new_zeros(b, h, capacity, d), "len": t}
        cache["k"][:, :, :t] = k
        cache["v"][:, :, :t] = v
        selected = torch.zeros(b, self.groups, capacity, device=k.device, dtype=torch.float32)
        selected[:, :, :t] = total.float()
        cache["selected"] = selected
        if live_keys:
            norms = torch.zeros(b, h, capacity, device=k.device, dtype=torch.float32)
            norms[:, :, :t] = kernels.key_norms(k)
            cache["key_norms"] = norms
        return y, cache

    def extend_cache(self, q, k, v, cache: dict, skip_dead_tiles: bool = False):
        """A further chunk of prompt tokens: (B, H, Tn, D) outputs in v's dtype; appends to the cache and moves
        ``selected`` on.  Equals the rows a single prefill over all tokens would produce.  ``skip_dead_tiles``: the
        part of the cache whose probabilities are all exactly zero for these queries is not read (same rows)."""
        return kernels.prefill_extend(cache, q, k, v, self.exempt, skip_dead_tiles=skip_dead_tiles).to(v.dtype)

    def step_cache(self, q1, k1, v1, cache: dict):
        """One token: (B, H, 1, D) in q1's dtype; appends to the cache and updates ``selected``."""
        if cache["len"] >= cache["k"].shape[2]:
            raise ValueError("decode step past the cache capacity (context_length)")
        if cache["k"].is_cuda and kernels.HAS_KERNELS and self.use_kernel:
            return kernels.decode_step(cache, q1, k1, v1, self.exempt).to(q1.dtype)
        raise RuntimeError("cached decode needs CUDA tensors and the built library (no CPU path)")
