"""Installs the unmodified reference project into ``baseline/_ref`` (git-ignored) and puts its own test files
(and the scripts folder one of them imports from) beside the package, so that a machine without the reference checkout can (a) run the reference's test suite
against this repository's drop-in module (``tests/test_reference_suite_gpu.py``) and (b) time the reference's own
code in ``bench.py --impl reference``.

    python baseline/install_reference.py /path/to/reference/checkout

Nothing from the reference enters this repository's history: ``baseline/_ref/`` is listed in ``.gitignore``.
The install is the offline pip recipe (no index, no build isolation) from a scratch copy of the checkout,
because the build writes an ``egg-info`` folder into the source tree it is given.
"""

from __future__ import annotations

import os
import shutil
import subprocess
import sys
import tempfile

HERE = os.path.dirname(os.path.abspath(__file__))
TARGET = os.path.join(HERE, "_ref")


def install(checkout: str) -> str:
    if not os.path.isdir(os.path.join(checkout, "src", "selective_attention")):
        raise SystemExit(f"{checkout} is not a checkout of the reference project")
    if os.path.isdir(TARGET):
        shutil.rmtree(TARGET)
    with tempfile.TemporaryDirectory() as tmp:
        copy = os.path.join(tmp, "reference")
        shutil.copytree(checkout, copy, ignore=shutil.ignore_patterns("runs", "results", "docs", ".git"))
        base = [sys.executable, "-m", "pip", "install", "--no-index", "--no-build-isolation", "--find-links",
                "/opt/wheelhouse", "--target", TARGET, "--quiet"]
        res = subprocess.run(base + [copy], stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
        if res.returncode != 0:        # dependency resolution against an empty index: the dependencies are in the image
            res = subprocess.run(base + ["--no-deps", copy], stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
        if res.returncode != 0:
            raise SystemExit("pip could not install the reference:\n" + res.stdout)
        for folder in ("tests", "scripts"):       # the tests import one helper from scripts/
            shutil.copytree(os.path.join(copy, folder), os.path.join(TARGET, folder))
    return TARGET


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit("usage: python baseline/install_reference.py /path/to/reference/checkout")
    print(install(sys.argv[1]))
