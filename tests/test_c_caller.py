"""The boundary from the other side: a plain C program (tests/c_caller/host_caller.c) that includes
include/gemm_b200.h, links libgemm_b200.so and nothing else of this repository.  Compiling it is a
CPU test (the header is valid C, every symbol it uses links); running it needs the GPU."""
import shutil
import subprocess
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
SRC = ROOT / "tests" / "c_caller" / "host_caller.c"


def _build(tmp_path):
    gcc = shutil.which("gcc")
    if gcc is None:
        pytest.skip("no gcc")
    exe = tmp_path / "host_caller"
    lib_dir = ROOT / "gemm_b200"
    cmd = [gcc, "-std=c11", "-O2", "-Wall", "-Wextra", "-Werror", "-I", str(ROOT / "include"), str(SRC), "-o", str(exe),
           "-L", str(lib_dir), "-lgemm_b200", f"-Wl,-rpath,{lib_dir}", "-lm"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    return exe


def test_header_is_plain_c_and_the_program_links(tmp_path):
    _build(tmp_path)


@pytest.mark.gpu
@pytest.mark.parametrize("M,K,N", [(64, 64, 64), (257, 100, 131)])
def test_c_program_gets_the_reference_bits(tmp_path, M, K, N):
    exe = _build(tmp_path)
    r = subprocess.run([str(exe), str(M), str(K), str(N)], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout + r.stderr
    assert r.stdout.startswith("ok ")
