"""Install the reference project's own attention package next to the oracle (TEST INFRASTRUCTURE).

    python -m oracle.build_ref [--source /path/to/reference/src]      (default: $PIPER_REF_SRC, then ../reference/src)

The reference (Boffee/piper-kernels) is pure Python: its ``piper_kernels.attention`` package holds
the portable quantized PyTorch loops (``attention/piper/reference.py``,
``attention/sage2pp/reference.py``) and the Triton kernels.  Its ``pyproject.toml`` names the
``uv_build`` backend, which is not available offline, so ``pip install --target`` cannot build
it; a pure-Python package's installed form is simply its files, and this recipe places them
under ``oracle/_ref/piper_kernels/`` where the reference tree is present.  ``oracle/_ref/`` is
git-ignored: nothing of it enters the history; it only travels with a working copy to a GPU box.

What may use it (and nothing else): ``tests/`` (a second, whole-tensor oracle: the reference's
own loop on CPU or CUDA tensors), ``bench.py --impl reference`` and the ``cpu_baseline`` leg
(the reference's CPU path on the host cores), and the reference-kernel timing script beside the
benchmark.  The product package never imports it.

``convrot`` is left out (another operator; it needs ``torchao``).
"""

from __future__ import annotations

import argparse
import os
import shutil
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
DEST = HERE / "_ref"
# where the reference's src/ directory is looked for: $PIPER_REF_SRC, then a checkout named
# "reference" beside this repository
DEFAULT_SOURCES = tuple(Path(x) for x in (os.environ.get("PIPER_REF_SRC"), HERE.parents[1] / "reference" / "src") if x)
PARTS = ("__init__.py", "attention", "_triton")


def find_source(explicit: str | None = None) -> Path | None:
    cands = [Path(explicit)] if explicit else list(DEFAULT_SOURCES)
    for c in cands:
        if (c / "piper_kernels" / "attention" / "piper" / "reference.py").exists():
            return c
    return None


def build(source: str | None = None, quiet: bool = False) -> Path | None:
    """Returns the install directory, or None when no reference tree is reachable (the prebuilt
    ``oracle/_ref`` of an earlier run, if any, is left as it is)."""
    src = find_source(source)
    if src is None:
        return DEST if (DEST / "piper_kernels").exists() else None
    pkg = DEST / "piper_kernels"
    if pkg.exists():
        shutil.rmtree(pkg)
    pkg.mkdir(parents=True)
    for part in PARTS:
        s = src / "piper_kernels" / part
        if s.is_dir():
            shutil.copytree(s, pkg / part, ignore=shutil.ignore_patterns("__pycache__", "*.pyc"))
        else:
            shutil.copy2(s, pkg / part)
    (DEST / "INSTALLED_FROM.txt").write_text(f"{src}\nparts: {', '.join(PARTS)}\n")
    if not quiet:
        print(f"reference attention package installed into {pkg}")
    return DEST


def import_reference():
    """Import the installed reference package; returns the module ``piper_kernels.attention`` or
    raises ImportError with the reason."""
    if not (DEST / "piper_kernels").exists():
        raise ImportError(f"{DEST}/piper_kernels is absent: run `python -m oracle.build_ref` where the reference tree exists")
    if str(DEST) not in sys.path:
        sys.path.insert(0, str(DEST))
    import importlib

    return importlib.import_module("piper_kernels.attention")


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--source", default=None)
    a = ap.parse_args()
    out = build(a.source)
    if out is None:
        print("no reference tree found; nothing installed")
