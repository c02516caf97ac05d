r"""Stages the reference's pure-Python package for the CPU baseline and the drop-in test.

    python oracle/stage_reference.py [/path/to/reference]

Copies ``fmoe/**/*.py`` and ``tests/moe.py`` of the reference checkout, unmodified, into
``baseline/_ref/`` (git-ignored: the reference's sources are not part of this repository;
the directory travels with the working tree to the GPU machine, where the checkout itself does
not exist).  Two users, both test infrastructure:

* ``bench.py --impl reference`` and the ``cpu_baseline`` leg import the reference's own
  ``NaiveGate`` (fmoe/gates/naive_gate.py:21-42) and ``BruteForceMoELinear`` (tests/moe.py:6-49)
  from there and time them on the host cores;
* ``tests/test_dropin_reference.py`` imports the reference's ``fmoe/functions.py`` with this
  library's ``fmoe_cuda`` module in place of the reference's extension.

The reference package imports ``fmoe_cuda`` at module load; callers install a module of that
name in ``sys.modules`` first (an empty one for the CPU path, which calls nothing in it).
"""
import os
import shutil
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DEST = os.path.join(ROOT, "baseline", "_ref")
DEFAULT_SRC = os.path.join(os.path.dirname(ROOT), "reference")


def stage(src=DEFAULT_SRC, dest=DEST):
    """Returns the destination directory, or None when the checkout is absent."""
    pkg = os.path.join(src, "fmoe")
    if not os.path.isdir(pkg):
        return None
    for base, _dirs, files in os.walk(pkg):
        rel = os.path.relpath(base, src)
        for f in files:
            if f.endswith(".py"):
                os.makedirs(os.path.join(dest, rel), exist_ok=True)
                shutil.copyfile(os.path.join(base, f), os.path.join(dest, rel, f))
    os.makedirs(os.path.join(dest, "tests"), exist_ok=True)
    shutil.copyfile(os.path.join(src, "tests", "moe.py"), os.path.join(dest, "tests", "moe.py"))
    return dest


def staged(dest=DEST):
    """Path of the staged copy if it is complete, else None."""
    ok = all(os.path.exists(os.path.join(dest, p)) for p in
             ("fmoe/__init__.py", "fmoe/functions.py", "fmoe/gates/naive_gate.py", "tests/moe.py"))
    return dest if ok else None


def import_reference(fmoe_cuda_module, dest=DEST):
    """Imports the staged reference package with ``fmoe_cuda_module`` standing in for its extension.
    Returns (fmoe package, moe test module) or None when nothing is staged."""
    if staged(dest) is None:
        return None
    import importlib
    for name in [n for n in sys.modules if n == "fmoe" or n.startswith("fmoe.") or n in ("moe", "fmoe_cuda")]:
        del sys.modules[name]
    sys.modules["fmoe_cuda"] = fmoe_cuda_module
    for p in (os.path.join(dest, "tests"), dest):
        if p not in sys.path:
            sys.path.insert(0, p)
    return importlib.import_module("fmoe"), importlib.import_module("moe")


if __name__ == "__main__":
    out = stage(sys.argv[1] if len(sys.argv) > 1 else DEFAULT_SRC)
    print(out if out else "reference checkout not found; nothing staged")
