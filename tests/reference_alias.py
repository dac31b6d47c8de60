"""pytest plugin (``-p reference_alias``) for running the reference project's own test files against this
repository's drop-in module: every ``selective_attention.kernels`` the reference's tests, layer and scripts import
becomes ``selective_attention_b200.kernels``.  The reference package itself (its model, config, runtime and the
frozen ``kernels_v1`` the suite cross-checks against) stays the installed, unmodified one."""

import sys

import selective_attention                      # the reference package (baseline/_ref on the path)
import selective_attention_b200.kernels as ours

sys.modules["selective_attention.kernels"] = ours
selective_attention.kernels = ours
for name in ("HAS_TRITON", "selective_attention", "selective_attention_forward", "selective_attention_reference",
             "selective_logits"):
    setattr(selective_attention, name, getattr(ours, name))
