"""Acceptance run of the drop-in boundary: the reference project's OWN test files
(``tests/test_selective_kernels.py``, ``test_selective_model.py``, ``test_selective_perhead.py``), unmodified,
executed with ``selective_attention.kernels`` replaced by ``selective_attention_b200.kernels``
(``tests/reference_alias.py``).  The reference's model, layer (``mixers.SelectiveAttention``), config and its frozen
``kernels_v1`` Triton kernels (one test cross-checks against them) are the installed originals.

The files come from ``baseline/_ref`` (``python baseline/install_reference.py``; git-ignored, it travels with the
working tree).  Without that folder the test is skipped with the command that creates it."""

import os
import re
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.path.join(ROOT, "baseline", "_ref")

pytestmark = pytest.mark.gpu


def test_reference_test_files_pass_against_the_drop_in_module():
    if not os.path.isdir(os.path.join(REF, "tests")):
        pytest.skip("baseline/_ref is missing: run `python baseline/install_reference.py <reference checkout>`")
    env = dict(os.environ)
    env["PYTHONPATH"] = os.pathsep.join([os.path.join(ROOT, "tests"), os.path.join(ROOT, "selective-attention-study_b200"),
                                         REF, env.get("PYTHONPATH", "")])
    cmd = [sys.executable, "-m", "pytest", "-p", "reference_alias", "-p", "no:cacheprovider", "-q", "-rfEs",
           "--rootdir", REF, "-c", os.devnull, os.path.join(REF, "tests")]
    res = subprocess.run(cmd, cwd=REF, env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=3000)
    tail = "\n".join(res.stdout.splitlines()[-40:])
    print(tail)
    log = os.environ.get("SA_PARITY_LOG")
    if log:
        with open(os.path.join(os.path.dirname(log), "reference_suite.log"), "w") as fh:
            fh.write(res.stdout)
    counts = {k: int(n) for n, k in re.findall(r"(\d+) (passed|failed|skipped|error|errors)", res.stdout.splitlines()[-1])}
    assert res.returncode == 0, tail
    assert counts.get("passed", 0) >= 100 and not counts.get("failed") and not counts.get("error"), tail
    assert counts.get("skipped", 0) == 0, tail            # on a GPU box nothing of the suite may skip
