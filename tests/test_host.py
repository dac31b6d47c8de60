"""CPU checks: the library loads and exports what the header declares; the Python boundary keeps the
reference's error contract; the dense listing in the package equals the oracle."""

import ctypes
import os
import re

import pytest
import torch

import selective_oracle as oracle
from selective_attention_b200 import _lib, kernels, mixers

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_functions():
    text = open(os.path.join(ROOT, "include", "selective_attention_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(sa_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    lib = _lib.load()
    declared = _declared_functions()
    assert set(_lib.EXPORTS) <= set(declared) and len(declared) >= 9
    for name in declared:
        assert hasattr(lib, name), name
    assert lib.sa_abi_version() == 3
    assert lib.sa_carry_rows(_lib.ENGINE_SIMT) == 32 and lib.sa_carry_rows(_lib.ENGINE_TCGEN05) == 128
    assert lib.sa_status_string(2) == b"unsupported shape, dtype or engine"


def test_problem_struct_matches_the_header_layout():
    assert ctypes.sizeof(_lib.Problem) == 10 * 4 + 9 * 8
    assert _lib.Problem.q_stride.offset == 40 and _lib.Problem.v_stride.offset == 88


def test_argument_checks_reject_before_any_launch():
    """No GPU needed: bad problems are refused with a status, never launched."""
    lib = _lib.load()
    p = _lib.Problem()
    assert lib.sa_backward_workspace_bytes(ctypes.byref(p)) == 0            # struct_bytes missing
    p.struct_bytes = ctypes.sizeof(_lib.Problem)
    p.dtype, p.engine, p.batch, p.heads, p.seq, p.head_dim, p.exempt = 0, 0, 1, 2, 64, 24, 1
    assert lib.sa_forward(ctypes.byref(p), 1, 1, 1, 1, 1, 1, 1, None) == 2  # head_dim 24
    p.head_dim, p.exempt = 32, 0
    assert lib.sa_forward(ctypes.byref(p), 1, 1, 1, 1, 1, 1, 1, None) == 1  # exempt 0
    p.exempt = 1
    assert lib.sa_forward(ctypes.byref(p), None, 1, 1, 1, 1, 1, 1, None) == 1  # null q
    need = lib.sa_backward_workspace_bytes(ctypes.byref(p))
    assert need >= 2 * 64 * 32 * 4 * 2
    assert lib.sa_decode_step(0, 1, 2, 1, 8, 8, 32, 1, 1, 1, 1, 1, 1, 1, 1, 1, 1 << 20, None) == 1  # cache full
    assert lib.sa_decode_step(0, 1, 2, 1, 7, 8, 32, 1, 16, 16, 16, 24, 16, 16, 16, 16, 1 << 20, None) == 3  # k_cache not 16-byte aligned
    # partial sums (rows x splits x (D + 2)), new selection (groups x t), tickets (rows + groups x splits)
    assert lib.sa_decode_workspace_bytes(1, 2, 1, 7, 32) == (2 * 1 * 34 + 8 + 2 + 1) * 4


def test_error_contract_on_cpu_tensors():
    q = torch.randn(1, 2, 64, 32)
    with pytest.raises(ValueError, match="CUDA"):
        kernels.selective_attention(q, q, q)
    with pytest.raises(ValueError, match="must all be"):
        kernels.selective_attention(q, q[:, :, :32], q)
    with pytest.raises(ValueError, match="exempt"):
        kernels.selective_attention_reference(q, q, q, exempt=0)
    with pytest.raises(TypeError):
        kernels.selective_attention_forward(q, q, q, None, None, 32, False, 4, None, None, 1, "linear")
    assert not kernels.supported(q) and not kernels.supported(q[..., :24])
    assert kernels.HEAD_DIMS == (16, 32, 64, 128) and torch.bfloat16 in kernels.DTYPES


def test_package_listing_equals_the_oracle(golden):
    g = golden("fb_b2_h3_t23_d16")
    torch.testing.assert_close(kernels.selective_attention_reference(g["q"], g["k"], g["v"]), g["out"],
                               atol=1e-5, rtol=1e-5)
    z, total = kernels.selective_logits(g["q"], g["k"])
    want_z, want_total = oracle.history_logits(g["q"], g["k"])
    torch.testing.assert_close(z, want_z)
    torch.testing.assert_close(total, g["total"], atol=1e-5, rtol=1e-5)


def test_slot_falls_back_to_the_listing_off_device_like_the_reference(golden):
    g = golden("fb_perhead")
    slot = mixers.SelectiveAttentionSlot.from_variant("selective_perhead", n_heads=4, context_length=64)
    y, total = slot.attend(g["q"], g["k"], g["v"], want_total=True)
    torch.testing.assert_close(y, g["out"], atol=1e-5, rtol=1e-5)
    torch.testing.assert_close(total, g["total"], atol=1e-5, rtol=1e-5)
    assert mixers.MIXER_TYPES == ("selective", "selective_x16", "selective_perhead")


def test_new_entry_points_check_their_arguments_before_any_launch():
    """Selector, layout-fused and prefill-continuation entry points refuse bad arguments with a status (no GPU)."""
    lib = _lib.load()
    p = _lib.Problem()
    p.struct_bytes = ctypes.sizeof(_lib.Problem)
    p.dtype, p.engine, p.batch, p.heads, p.seq, p.head_dim, p.exempt = 1, 1, 1, 2, 256, 64, 1
    sel = _lib.Selector()                                        # struct_bytes missing
    assert lib.sa_forward_selector(ctypes.byref(p), 16, 16, 16, ctypes.byref(sel), 16, 16, 16, 16, None) == 1
    sel.struct_bytes = ctypes.sizeof(_lib.Selector)              # null q0 / k0
    assert lib.sa_forward_selector(ctypes.byref(p), 16, 16, 16, ctypes.byref(sel), 16, 16, 16, 16, None) == 1
    assert ctypes.sizeof(_lib.Selector) == 8 + 2 * 8 + 4 * 8 and ctypes.sizeof(_lib.Tensor) == 8 + 8 + 3 * 8
    low = _lib.Tensor()
    low.ptr, low.dtype = 16, 0                                   # fp32 descriptor for a bf16 problem
    low.stride[:] = [64 * 256 * 2, 64, 128]
    assert lib.sa_forward_fused(ctypes.byref(p), 16, 16, 16, None, 16, ctypes.byref(low), 16, 16, 16, None) == 1
    low.dtype = 1
    low.stride[:] = [64 * 256 * 2, 64, 100]                      # token stride of 200 bytes: rows not 16-byte aligned
    assert lib.sa_forward_fused(ctypes.byref(p), 16, 16, 16, None, 16, ctypes.byref(low), 16, 16, 16, None) == 3
    p.engine = 0                                                 # the CUDA-core engine has no fused or continuation form
    low.stride[:] = [64 * 256 * 2, 64, 128]
    assert lib.sa_forward_fused(ctypes.byref(p), 16, 16, 16, None, 16, ctypes.byref(low), 16, 16, 16, None) == 2
    assert lib.sa_prefill_extend(ctypes.byref(p), 128, 16, 16, 16, 16, 256, 16, 16, 16, 16, None) == 2
    p.engine = 1
    assert lib.sa_prefill_extend(ctypes.byref(p), 256, 16, 16, 16, 16, 256, 16, 16, 16, 16, None) == 1   # nothing new
    assert lib.sa_prefill_extend(ctypes.byref(p), 128, 16, 16, 16, 16, 100, 16, 16, 16, 16, None) == 1   # selected too short
    assert lib.sa_selection_carry(ctypes.byref(p), 16, 16, None, 16, 16, None) == 2                      # CUDA-core engine only
    assert lib.sa_selftest_wait_timeout(0, None) == 1
    assert lib.sa_launch_count() >= 0


def test_live_tile_entry_points_check_their_arguments_before_any_launch():
    """The table of live tiles: its size, and the refusals that need no GPU."""
    lib = _lib.load()
    p = _lib.Problem()
    p.struct_bytes = ctypes.sizeof(_lib.Problem)
    p.dtype, p.engine, p.batch, p.heads, p.seq, p.head_dim, p.exempt = 1, 1, 2, 3, 1000, 64, 1
    nt, rows = 8, 6
    table = (rows * nt * nt + 255) // 256 * 256
    assert lib.sa_tile_table_bytes(ctypes.byref(p)) == table + 2 * rows * nt * 4      # verdicts + the two norm arrays
    p.seq = 131072 + 1                                           # more than 1024 key tiles: not offered
    assert lib.sa_tile_table_bytes(ctypes.byref(p)) == 0
    p.seq, p.head_dim = 1000, 32
    assert lib.sa_tile_table_bytes(ctypes.byref(p)) == 0        # tensor-core shapes only
    p.head_dim, p.engine = 64, 0
    assert lib.sa_tile_table_bytes(ctypes.byref(p)) == 0        # CUDA-core engine
    args = (16, 16, 16, None, 16, None, 16, 16, 16)
    assert lib.sa_forward_live_tiles(ctypes.byref(p), *args, 256, 1 << 20, None) == 2
    p.engine = 1
    assert lib.sa_forward_live_tiles(ctypes.byref(p), *args, 256, 16, None) == 4      # table too small
    assert lib.sa_forward_live_tiles(ctypes.byref(p), *args, 16, 1 << 20, None) == 3  # table not 256-byte aligned
    # the decode step with key norms refuses what the plain step refuses (here: a full cache)
    assert lib.sa_decode_step_live_keys(0, 1, 2, 1, 8, 8, 32, 1, 1, 1, 1, 1, 1, 1, 1, 1, 1, 1 << 20, None) == 1
    cont = (128, 16, 16, 16, 16, 1000, 16, 16, 16, 16)
    assert lib.sa_prefill_extend_live_tiles(ctypes.byref(p), *cont, 256, 16, None) == 4   # table too small
    assert lib.sa_prefill_extend_live_tiles(ctypes.byref(p), *cont, 16, 1 << 20, None) == 3


def test_selector_and_packed_arguments_are_validated_in_python():
    q = torch.randn(1, 2, 64, 64)
    with pytest.raises(ValueError, match="CUDA"):
        kernels.selective_attention(q, q, q, selector=(q[:, 0], q[:, 0]))
    assert not kernels.packed_supported(torch.randn(1, 64, 3, 2, 64))          # CPU, fp32
    with pytest.raises(ValueError, match="contiguous bf16 CUDA"):
        kernels.selective_attention_packed(torch.randn(1, 64, 3, 2, 64))
    with pytest.raises(ValueError, match="carry_rows"):
        kernels._carry_rows_request(64)
    assert kernels._carry_rows_request(None) is None and kernels._carry_rows_request(32) == 32
