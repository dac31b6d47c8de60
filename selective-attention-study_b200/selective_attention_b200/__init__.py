"""B200-native Selective Attention operator (drop-in for the reference's ``selective_attention.kernels``)."""

from .kernels import (CARRY_M, DTYPES, HAS_KERNELS, HAS_TRITON, HEAD_DIMS, check_inputs, decode_step,
                      selective_attention, selective_attention_forward, selective_attention_reference,
                      selective_logits, supported)

__all__ = ["CARRY_M", "DTYPES", "HAS_KERNELS", "HAS_TRITON", "HEAD_DIMS", "check_inputs", "decode_step",
           "selective_attention", "selective_attention_forward", "selective_attention_reference",
           "selective_logits", "supported"]
