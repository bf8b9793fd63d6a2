"""The bounds-checking build of the library (-DGEMM_B200_DEBUG): ragged shapes run clean, and the
checks do fire — shown by telling the checker that every matrix is a little shorter than it is, so
that it refuses (and skips) accesses that are in fact inside the matrix.  No access ever leaves a
matrix in either run.  Each run is a child process because the library is chosen at load time."""
import os
import subprocess
import sys
from pathlib import Path

import pytest

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parents[1]
DEBUG_LIB = ROOT / "gemm_b200" / "profiling" / "libgemm_b200_debug.so"


def _run(*args):
    assert DEBUG_LIB.exists(), "python -m gemm_b200.build builds it"
    env = dict(os.environ, GEMM_B200_LIB=str(DEBUG_LIB))
    return subprocess.run([sys.executable, "-m", "gemm_b200.profiling.run_bounds", *args], cwd=ROOT, env=env,
                          capture_output=True, text=True, timeout=600)


def test_ragged_shapes_are_clean():
    r = _run()
    assert r.returncode == 0, r.stdout + r.stderr
    assert "refused" not in r.stdout and r.stdout.count("clean") >= 7


def test_understated_extents_are_refused_not_accessed():
    r = _run("--shrink", "64")
    assert r.returncode == 0, r.stdout + r.stderr
    assert "clean" not in r.stdout and r.stdout.count("refused at site") >= 7
