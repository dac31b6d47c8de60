"""Known-answer test of the tcgen05 / TMA operand encodings (exact integer data, zero error expected)."""

import pytest
import torch

from selective_attention_b200 import _lib

pytestmark = pytest.mark.gpu


def test_tcgen05_operand_forms_are_exact():
    lib = _lib.load()
    scratch = torch.zeros(64 * 1024, dtype=torch.uint8, device="cuda")
    assert scratch.data_ptr() % 1024 == 0
    result = torch.full((8,), -1.0, device="cuda")
    _lib.check("sa_selftest_tcgen05", lib.sa_selftest_tcgen05(scratch.data_ptr(), result.data_ptr(), None))
    torch.cuda.synchronize()
    assert _lib.device_status() == 0
    got = result[:5].cpu().tolist()
    assert got == [0.0] * 5, got
