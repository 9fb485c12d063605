"""Stages the reference's three attention test modules, unmodified, for a run against this build.

TEST INFRASTRUCTURE ONLY.  The reference's callers for the attention path are its own pytest files
(tests/test_attention.py, tests/test_decode.py, tests/test_speculative_decode.py); they import
``kernels.attention`` / ``kernels`` by name and compare with fp32 SDPA on a CUDA device.  A reference
checkout does not exist on a GPU machine, so this recipe copies those three files byte for byte into
``oracle/_ref/tests/`` (git-ignored: reference sources never enter this repository's history) from
where ``tests/test_zr_reference_suite.py`` runs them with this build's package first on PYTHONPATH.

    python oracle/stage_reference_tests.py [path-to-reference-checkout]
"""
import hashlib
import os
import shutil
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
DEST = os.path.join(HERE, "_ref", "tests")
FILES = ("test_attention.py", "test_decode.py", "test_speculative_decode.py")


def default_checkout() -> str:
    """``$B200ATTN_REFERENCE_CHECKOUT``, else a directory named ``reference`` beside this repository."""
    repo = os.path.dirname(HERE)
    return os.environ.get("B200ATTN_REFERENCE_CHECKOUT", os.path.join(os.path.dirname(repo), "reference"))


def stage(ref_root: str = "") -> bool:
    """Returns False (and stages nothing) when there is no reference checkout at ``ref_root``."""
    ref_root = ref_root or default_checkout()
    src_dir = os.path.join(ref_root, "tests")
    if not all(os.path.isfile(os.path.join(src_dir, f)) for f in FILES):
        return False
    os.makedirs(DEST, exist_ok=True)
    lines = []
    for f in FILES:
        dst = os.path.join(DEST, f)
        shutil.copyfile(os.path.join(src_dir, f), dst)
        with open(dst, "rb") as fh:
            lines.append(f"{hashlib.sha256(fh.read()).hexdigest()}  {f}\n")
    with open(os.path.join(DEST, "SHA256SUMS"), "w") as fh:
        fh.writelines(lines)
    return True


if __name__ == "__main__":
    ok = stage(sys.argv[1] if len(sys.argv) > 1 else "")
    print("staged into", DEST if ok else "nothing: no reference checkout found")
