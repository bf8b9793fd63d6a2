"""The reference's own test.py and benchmark.py, unchanged, against this repository's variant
directories (no GPU needed: the check is that they import, i.e. that their two-file
torch.utils.cpp_extension.load() call builds our sources and yields a module with the function
they go on to call).

The scripts are read from a checkout of the reference ($GEMM_B200_REFERENCE, else a `reference`
folder beside this repository) and are never copied; where there is no checkout the test is
skipped.  Each script names its sources relative to the working directory (naive/test.py:7), so
running it with the working directory in gemm_b200/variants/<variant>/ makes it build ours."""
import os
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
REF = Path(os.environ.get("GEMM_B200_REFERENCE") or (ROOT.parent / "reference"))

# variant -> (attribute the script binds the module to, function it calls)
VARIANTS = {
    "naive": ("naive_gemm_cuda", "naive_gemm"),          # naive/test.py:5,22
    "shared": ("custom_gemm", "gemm_cuda"),              # shared/test.py:5,27
    "blocktile_1d": ("custom_gemm", "gemm_cuda"),        # blocktile_1d/test.py:5,27
}

CHILD = r"""
import importlib.util, sys
ref, variant, attr, fn = sys.argv[1:5]
for script in ("test.py", "benchmark.py"):
    spec = importlib.util.spec_from_file_location("ref_%s_%s" % (variant, script[:-3]), "%s/%s/%s" % (ref, variant, script))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)                 # runs the script's load(...) with cwd = our variant directory
    ext = getattr(mod, attr)
    assert callable(getattr(ext, fn)), (script, fn)
    assert callable(getattr(ext, "matmul"))      # our additive two-argument form
print("ok", variant)
"""


@pytest.mark.skipif(not (REF / "naive" / "test.py").exists(), reason="no checkout of the reference on this machine")
def test_reference_scripts_import_unchanged_from_our_variant_directories(tmp_path):
    procs = {}
    for variant, (attr, fn) in VARIANTS.items():
        env = dict(os.environ, TORCH_EXTENSIONS_DIR=str(tmp_path / variant), TORCH_CUDA_ARCH_LIST="10.0", MAX_JOBS="4")
        procs[variant] = subprocess.Popen([sys.executable, "-c", CHILD, str(REF), variant, attr, fn],
                                          cwd=ROOT / "gemm_b200" / "variants" / variant, env=env,
                                          stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    for variant, p in procs.items():
        out, _ = p.communicate(timeout=900)
        assert p.returncode == 0, out[-3000:]
        assert ("ok " + variant) in out
