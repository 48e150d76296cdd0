"""Recipe for ``oracle/_ref``: an unmodified copy of the reference project's own Python package, taken from
its checkout, for use as the CPU arm of the benchmark (``bench.py --impl reference`` and ``cpu_baseline``)
and as a cross-check of the oracle.

    python oracle/make_ref.py [/path/to/reference]

Only the package directory ``python/adangel`` is copied (pure Python: its semantic reference
``adangel.reference.run_o{0,1,2}_reference``, codecs and schema).  ``oracle/_ref/`` is git-ignored: nothing of
the reference enters this repository's history.  Test infrastructure: the product never imports it.
"""

from __future__ import annotations

import shutil
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
DEFAULT_REFERENCE = Path("/root/reference")


def make_ref(reference_root=DEFAULT_REFERENCE) -> Path | None:
    """Copies the package and returns its parent directory (to be put on ``sys.path``), or None when the
    checkout is not present (an existing copy is then left as it is)."""
    source = Path(reference_root) / "python" / "adangel"
    target = HERE / "_ref"
    if not source.is_dir():
        return target if (target / "adangel").is_dir() else None
    if (target / "adangel").exists():
        shutil.rmtree(target / "adangel")
    target.mkdir(exist_ok=True)
    shutil.copytree(source, target / "adangel", ignore=shutil.ignore_patterns("__pycache__", "*.pyc", "*.so"))
    (target / "SOURCE.txt").write_text(f"copied unmodified from {source}\n", encoding="utf-8")
    return target


if __name__ == "__main__":
    print(make_ref(sys.argv[1] if len(sys.argv) > 1 else DEFAULT_REFERENCE))
