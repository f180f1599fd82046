"""Installs the unmodified reference project into ``baseline/_ref`` (offline).

The reference ships no ``setup.py`` / ``pyproject.toml``, so a plain
``pip install --target baseline/_ref <reference>`` fails ("not installable").  This script
copies the reference to a temporary directory, adds a packaging stub that lists its
top-level modules (no source file is touched), installs that copy with ``--no-deps`` and
verifies that the installed modules are byte-identical to the reference's.

    python baseline/install_reference.py [/path/to/reference] [--find-links DIR]

The wheel directory pip may look into comes from ``--find-links``, else from the
``PIP_FIND_LINKS`` environment variable; with neither, pip is run without one (the install
needs no wheels: it uses ``--no-deps``).
"""
from __future__ import annotations

import filecmp
import os
import shutil
import subprocess
import sys
import tempfile
from pathlib import Path

HERE = Path(__file__).resolve().parent
TARGET = HERE / "_ref"
MODULES = ["baseline", "utils", "benchmark", "kernels", "unit_tests"]

STUB = '''from setuptools import setup
# Packaging metadata only: the reference ships no build files.
setup(name="iris_testing_reference", version="0.0.0", py_modules=%r)
''' % (MODULES,)


def install(reference: Path, find_links: str | None = None) -> str | None:
    """Returns None on success, else a one-line reason."""
    if not (reference / "baseline.py").exists():
        return f"no reference tree at {reference}"
    links = find_links or os.environ.get("PIP_FIND_LINKS")
    pip = [sys.executable, "-m", "pip", "install", "--no-index", "--no-build-isolation"]
    if links:
        pip += ["--find-links", links.split()[0]]
    pip += ["--target", str(TARGET)]
    first = subprocess.run(pip + [str(reference)], capture_output=True, text=True)
    if first.returncode != 0:
        with tempfile.TemporaryDirectory() as tmp:
            copy = Path(tmp) / "reference"
            shutil.copytree(reference, copy)
            for p in copy.rglob("*"):
                p.chmod(p.stat().st_mode | 0o200)
            copy.chmod(copy.stat().st_mode | 0o200)
            (copy / "setup.py").write_text(STUB)
            second = subprocess.run(pip + ["--no-deps", "--upgrade", str(copy)], capture_output=True,
                                    text=True, cwd=str(copy))
            if second.returncode != 0:
                return ("pip install failed: " + (second.stderr.strip().splitlines() or ["?"])[-1])[:200]
    for m in MODULES:
        if not filecmp.cmp(reference / f"{m}.py", TARGET / f"{m}.py", shallow=False):
            return f"installed {m}.py differs from the reference"
    return None


if __name__ == "__main__":
    argv = sys.argv[1:]
    links = None
    if "--find-links" in argv:
        i = argv.index("--find-links")
        links = argv[i + 1]
        del argv[i:i + 2]
    ref = Path(argv[0]) if argv else HERE.parent.parent / "reference"
    err = install(ref, links)
    print("ok" if err is None else f"failed: {err}")
    sys.exit(0 if err is None else 1)
