"""Places an unmodified copy of the reference project under ``baseline/_ref/``.

    SPCONV_REFERENCE_ROOT=/path/to/spconv-triton python baseline/install_reference.py

``pip install`` of the reference cannot work offline here (its build backend,
hatchling, is not installed), and the package is pure Python, so a plain copy
of the source tree (package + tests + test data) is the install.  The copy is
git-ignored; it is used by ``bench.py --op reference_gpu`` / ``--op published``
(the reference's Triton kernels timed on the same GPU) and by
``tests/test_gpu_reference_suite.py`` (the reference's own test files run
against this package).  Nothing of the product imports it.
"""

from __future__ import annotations

import os
import shutil
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
DEST = HERE / "_ref" / "reference"


def main() -> int:
    src = os.environ.get("SPCONV_REFERENCE_ROOT")
    if not src or not (Path(src) / "spconv_triton").is_dir():
        print("set SPCONV_REFERENCE_ROOT to a checkout of the reference project", file=sys.stderr)
        return 1
    if DEST.exists():
        shutil.rmtree(DEST)
    shutil.copytree(src, DEST, ignore=shutil.ignore_patterns(".git", "__pycache__", "*.pyc", ".pytest_cache"))
    print(DEST)
    return 0


if __name__ == "__main__":
    sys.exit(main())
