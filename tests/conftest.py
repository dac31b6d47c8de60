"""Test configuration: puts the package and the oracle on the import path and registers the
``gpu`` marker (tests that need a B200; everything else runs on the CPU)."""

import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for sub in ("selective-attention-study_b200", "oracle", ""):
    path = os.path.join(ROOT, sub)
    if path not in sys.path:
        sys.path.insert(0, path)

GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def golden():
    import numpy as np
    import torch

    def load(name):
        with np.load(os.path.join(GOLDEN, name + ".npz")) as data:
            return {k: (torch.from_numpy(data[k]) if data[k].ndim else data[k].item()) for k in data.files}

    return load


@pytest.fixture(scope="session")
def achieved():
    """Records the error a parity test achieved (not only that it was under its bar): prints it, so it shows
    with ``pytest -rP`` / ``-s``, and appends a JSON line to the file named by SA_PARITY_LOG when that is set."""
    import json

    def record(case: str, **values):
        line = {"case": case, **{k: (float(v) if v is not None else None) for k, v in values.items()}}
        print("achieved:", json.dumps(line))
        path = os.environ.get("SA_PARITY_LOG")
        if path:
            with open(path, "a") as fh:
                fh.write(json.dumps(line) + "\n")

    return record
