"""Runs the reference's own attention test modules, byte for byte as the reference ships them,
against this build's ``kernels`` package on the GPU.

The reference's callers for this path are its pytest files (tests/test_attention.py:8,137-251,
tests/test_decode.py:8,133-244, tests/test_speculative_decode.py:8,169-332): they import
``kernels.attention.flash_attention_v2``, ``kernels.decode_attention`` and
``kernels.speculative_decode_attention`` by name.  ``oracle/stage_reference_tests.py`` stages the three files
(git-ignored) where this test finds them; their digests are checked so "unmodified" is a tested fact."""
import hashlib
import os
import re
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
STAGED = os.path.join(ROOT, "oracle", "_ref", "tests")
PKG = os.path.join(ROOT, "triton-kernels_b200")

# sha256 of the reference's files at the commit this build was made against
DIGESTS = {
    "test_attention.py": "bc3cd14a8ca12ac7db6a6cce12d2c1f162758c1cfefb9b725c0c0a0778f4475b",
    "test_decode.py": "75a76bbb1c0f5001fef68faeb9cf566b8c54abb594339d9ed3151490d1136319",
    "test_speculative_decode.py": "491802214603d819874263465e638fc9310e4333ad2b1c72ed2d09af7c295dec",
}
# cases the reference's parametrisation yields: 108 prefill (27 causal+cross skipped by the reference itself),
# 27 decode, 432 speculative decode
EXPECT = {"test_attention.py": (81, 27), "test_decode.py": (27, 0), "test_speculative_decode.py": (432, 0)}


def _staged():
    return all(os.path.isfile(os.path.join(STAGED, f)) for f in DIGESTS)


@pytest.mark.gpu
@pytest.mark.parametrize("module", sorted(DIGESTS))
def test_reference_module_passes_unmodified(module):
    if not _staged():
        pytest.skip("reference test modules not staged: run `python oracle/stage_reference_tests.py` where a "
                    "reference checkout exists")
    path = os.path.join(STAGED, module)
    with open(path, "rb") as fh:
        assert hashlib.sha256(fh.read()).hexdigest() == DIGESTS[module], f"{module} differs from the reference's file"
    env = dict(os.environ)
    env["PYTHONPATH"] = PKG + os.pathsep + env.get("PYTHONPATH", "")
    # run from the staging directory with no ini file and no conftest of this repository in reach
    proc = subprocess.run(
        [sys.executable, "-m", "pytest", module, "-q", "-p", "no:cacheprovider", "--rootdir", STAGED, "-c", os.devnull,
         "--noconftest"],
        cwd=STAGED, env=env, capture_output=True, text=True, timeout=1500)
    tail = proc.stdout[-3000:] + proc.stderr[-2000:]
    out_dir = os.environ.get("B200ATTN_TEST_LOG_DIR", "")      # optional: keep each module's pytest output there
    if out_dir and os.path.isdir(out_dir):
        with open(os.path.join(out_dir, "reference_suite_" + module.replace(".py", ".log")), "w") as fh:
            fh.write(proc.stdout[-20000:] + proc.stderr[-5000:])
    assert proc.returncode == 0, tail
    passed = int((re.search(r"(\d+) passed", proc.stdout) or [0, 0])[1])
    skipped = int((re.search(r"(\d+) skipped", proc.stdout) or [0, 0])[1])
    failed = re.search(r"(\d+) (failed|error)", proc.stdout)
    assert failed is None, tail
    assert (passed, skipped) == EXPECT[module], f"{module}: {passed} passed / {skipped} skipped, expected {EXPECT[module]}\n{tail}"
