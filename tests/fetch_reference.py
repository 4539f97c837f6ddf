"""Puts a copy of the reference checkout where the GPU tests and `bench.py --impl reference` look
for it:

    python tests/fetch_reference.py [/path/to/reference]      (default: ../reference)

copies the reference's `switchyard/` package and its `tests/tiny.py` helper, unchanged, into
`baseline/_ref/` of this repository. That folder is ignored by git (nothing of the reference is
committed) but travels with the working tree to machines that have no reference checkout. The
drop-in tests (tests/test_dropin_gpu.py) import the reference's own `model.py` / `serve.py` from
there and run them on this package's kernels; they skip when the folder is absent."""

import os
import shutil
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DEST = os.path.join(ROOT, "baseline", "_ref")


def fetch(src):
    pkg = os.path.join(src, "switchyard")
    if not os.path.exists(os.path.join(pkg, "moe.py")):
        raise SystemExit(f"{src} does not look like a checkout of the reference (no switchyard/moe.py)")
    if os.path.exists(DEST):
        shutil.rmtree(DEST)
    os.makedirs(DEST)
    shutil.copytree(pkg, os.path.join(DEST, "switchyard"), ignore=shutil.ignore_patterns("__pycache__"))
    os.makedirs(os.path.join(DEST, "tests"))
    shutil.copy(os.path.join(src, "tests", "tiny.py"), os.path.join(DEST, "tests", "tiny.py"))
    return DEST


if __name__ == "__main__":
    print(fetch(sys.argv[1] if len(sys.argv) > 1 else os.path.join(os.path.dirname(ROOT), "reference")))
