"""Stages the reference project's own hot-path test files for the drop-in check.

The reference (TheTom/turboquant_plus) ships ten test files for the path this library replaces
(tests/test_{rotation,codebook,polar_quant,qjl,turboquant,kv_cache,utils,turbo4,distortion,outlier}.py).  They are
the acceptance suite of the drop-in claim: the same files, unmodified, run against ``turboquant_plus_b200`` aliased
as ``turboquant`` (tests/reference_suite/conftest.py).  The files are NOT part of this repository: this script copies
them from a checkout of the reference into ``tests/reference_suite/_ref/`` (ignored by git), so that they can travel
to a machine that has a GPU but no checkout.

    python tests/reference_suite/stage.py [path of the reference checkout]

Without an argument the checkout is looked for in $TQ_REFERENCE_DIR, then in a directory ``reference`` beside the
repository.  Returns quietly when there is none (the suite is then reported as skipped).
"""
import os
import shutil
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
REPO = os.path.dirname(os.path.dirname(HERE))
DEST = os.path.join(HERE, "_ref")
FILES = ["test_rotation.py", "test_codebook.py", "test_polar_quant.py", "test_qjl.py", "test_turboquant.py",
         "test_kv_cache.py", "test_utils.py", "test_turbo4.py", "test_distortion.py", "test_outlier.py"]


def reference_dir(arg=None):
    for cand in (arg, os.environ.get("TQ_REFERENCE_DIR"), os.path.join(os.path.dirname(REPO), "reference")):
        if cand and os.path.isdir(os.path.join(cand, "tests")) and os.path.isdir(os.path.join(cand, "turboquant")):
            return cand
    return None


def stage(arg=None) -> int:
    """Copies the ten files; returns how many are in place afterwards."""
    ref = reference_dir(arg)
    if ref is None:
        return len([f for f in FILES if os.path.exists(os.path.join(DEST, f))])
    os.makedirs(DEST, exist_ok=True)
    for f in FILES:
        shutil.copyfile(os.path.join(ref, "tests", f), os.path.join(DEST, f))
    open(os.path.join(DEST, "__init__.py"), "a").close()
    return len(FILES)


if __name__ == "__main__":
    n = stage(sys.argv[1] if len(sys.argv) > 1 else None)
    print(f"{n} of {len(FILES)} reference test files in {DEST}")
