"""In-tree build of the native parts: `python -m gemm_b200.build [--variants] [--force]`.

Produces, next to the sources (all git-ignored, all shipped with the working tree):

* ``gemm_b200/libgemm_b200.so`` — the C-ABI library declared in ``include/gemm_b200.h``
  (FP32 CUDA-core kernels + sm_100a tensor-core kernels), built with nvcc for
  ``arch=compute_100a,code=sm_100a``;
* ``gemm_b200/profiling/libgemm_b200_probe.so`` — the TMA streaming probe (a measurement helper,
  not part of the GEMM library);
* ``gemm_b200/profiling/libgemm_b200_trace.so`` — the library compiled with its opt-in stage
  timeline (``-DGEMM_B200_TRACE``), for ``python -m gemm_b200.profiling.run_trace``;
* ``gemm_b200/profiling/libgemm_b200_debug.so`` — the bounds-checking build (``-DGEMM_B200_DEBUG``);
* ``gemm_b200/variants/<variant>/<module>.so`` — one PyTorch extension module per reference
  variant, with the reference's module and function names
  (naive/test.py:5-11, shared/test.py:5-11, blocktile_1d/test.py:5-11).

Every step is skipped when its output is newer than its inputs.
"""
from __future__ import annotations

import argparse
import concurrent.futures as cf
import os
import shutil
import subprocess
import sys
import sysconfig
from pathlib import Path

PKG = Path(__file__).resolve().parent
ROOT = PKG.parent
CSRC = PKG / "csrc"
INCLUDE = ROOT / "include"
BUILD = PKG / "build"
LIB = PKG / "libgemm_b200.so"
PROBE_LIB = PKG / "profiling" / "libgemm_b200_probe.so"

ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_COMMON = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC"]
# host-side warnings are errors (the device front end's own diagnostics stay warnings)
HOST_WARNINGS = ["-Xcompiler", "-Wall,-Wextra,-Werror,-Wno-unused-parameter"]

# translation unit -> extra flags.  The FP32 kernel flushes denormals like the reference, which
# is built with --use_fast_math (naive/test.py:8).
LIB_SOURCES = {
    "sgemm_f32.cu": ["-ftz=true"],
    "tc_gemm.cu": [],
    "status.cu": [],
    "host_api.cu": [],
}

# variant dir -> (module name, [cpp, cu]) — the names the reference's scripts pass to load()
VARIANTS = {
    "naive": ("naive_gemm_cuda", ["naive.cpp", "naive_1.cu"]),
    "shared": ("shared_gemm", ["shared.cpp", "shared_2.cu"]),
    "blocktile_1d": ("blocktile_1d", ["blocktile_1d.cpp", "blocktile_1d.cu"]),
}


# `python -m gemm_b200.build --tuning` also compiles the kernel variants the heuristics never pick
TUNING: list[str] = []


def nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(exe).exists():
        raise RuntimeError("nvcc not found; the gemm_b200 native library cannot be built")
    return exe


def _newer(out: Path, deps: list[Path]) -> bool:
    if not out.exists():
        return False
    t = out.stat().st_mtime
    return all(d.stat().st_mtime <= t for d in deps if d.exists())


def _run(cmd: list[str], cwd: Path | None = None) -> None:
    proc = subprocess.run(cmd, cwd=cwd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if proc.returncode != 0:
        raise RuntimeError("command failed: %s\n%s" % (" ".join(cmd), proc.stdout))


def _headers() -> list[Path]:
    return sorted(CSRC.glob("*.cuh")) + sorted(INCLUDE.glob("*.h"))


def build_library(force: bool = False, verbose: bool = False) -> Path:
    BUILD.mkdir(exist_ok=True)
    hdrs = _headers()
    jobs = []
    objs = []
    for src, extra in LIB_SOURCES.items():
        s = CSRC / src
        o = BUILD / (s.stem + ".o")
        objs.append(o)
        if force or not _newer(o, [s] + hdrs):
            cmd = [nvcc(), *ARCH, *NVCC_COMMON, *HOST_WARNINGS, *extra, *TUNING, "-c", str(s), "-o", str(o)]
            if verbose:
                cmd.insert(1, "-Xptxas=-v")
            jobs.append(cmd)
    if jobs:
        with cf.ThreadPoolExecutor(max_workers=len(jobs)) as ex:
            list(ex.map(_run, jobs))
    if force or jobs or not _newer(LIB, objs):
        _run([nvcc(), *ARCH, "-shared", "-o", str(LIB), *map(str, objs)])
    return LIB


def build_probe(force: bool = False) -> Path:
    """The TMA streaming probe of gemm_b200.profiling, a shared library of its own."""
    src = PKG / "profiling" / "probe_tma_stream.cu"
    if force or not _newer(PROBE_LIB, [src] + _headers()):
        _run([nvcc(), *ARCH, *NVCC_COMMON, *HOST_WARNINGS, "-shared", str(src), "-o", str(PROBE_LIB)])
    return PROBE_LIB


def build_debug(force: bool = False) -> Path:
    """The bounds-checking build (-DGEMM_B200_DEBUG): gemm_b200/profiling/libgemm_b200_debug.so.  Every
    access the kernels address themselves is checked against its matrix first; one that falls
    outside is skipped and recorded (GEMM_B200_ERR_BOUNDS), never made.  Load it with GEMM_B200_LIB."""
    return _build_flavour("debug", "-DGEMM_B200_DEBUG", force)


def build_trace(force: bool = False) -> Path:
    """The library with the stage timeline compiled in (-DGEMM_B200_TRACE), for gemm_b200.profiling.run_trace:
    gemm_b200/profiling/libgemm_b200_trace.so.  Load it with GEMM_B200_LIB=<that path>."""
    return _build_flavour("trace", "-DGEMM_B200_TRACE", force)


def _build_flavour(name: str, define: str, force: bool) -> Path:
    out = PKG / "profiling" / f"libgemm_b200_{name}.so"
    if not force and _newer(out, [CSRC / src for src in LIB_SOURCES] + _headers()):
        return out
    bdir = BUILD / name
    bdir.mkdir(parents=True, exist_ok=True)
    objs, jobs = [], []
    for src, extra in LIB_SOURCES.items():
        o = bdir / (Path(src).stem + ".o")
        objs.append(o)
        jobs.append([nvcc(), *ARCH, *NVCC_COMMON, *HOST_WARNINGS, *extra, define, "-c", str(CSRC / src), "-o", str(o)])
    with cf.ThreadPoolExecutor(max_workers=len(jobs)) as ex:
        list(ex.map(_run, jobs))
    _run([nvcc(), *ARCH, "-shared", "-o", str(out), *map(str, objs)])
    return out


def _torch_flags() -> tuple[list[str], list[str]]:
    from torch.utils import cpp_extension as ce

    inc = ["-I" + p for p in ce.include_paths()] + ["-I" + sysconfig.get_paths()["include"]]
    libdirs = ce.library_paths()
    ld = ["-L" + p for p in libdirs] + ["-Wl,-rpath," + p for p in libdirs]
    ld += ["-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch", "-ltorch_python"]
    return inc, ld


def variant_module_path(variant: str) -> Path:
    name, _ = VARIANTS[variant]
    return PKG / "variants" / variant / (name + ".so")


def build_variant(variant: str, force: bool = False) -> Path:
    """Builds one reference-named extension module with plain g++/nvcc (no JIT cache)."""
    name, (cpp, cu) = VARIANTS[variant]
    vdir = PKG / "variants" / variant
    out = variant_module_path(variant)
    deps = [vdir / cpp, vdir / cu, CSRC / "sgemm_f32.cu", CSRC / "status.cu"] + _headers()
    if not force and _newer(out, deps):
        return out
    inc, ld = _torch_flags()
    bdir = BUILD / variant
    bdir.mkdir(parents=True, exist_ok=True)
    defs = ["-DTORCH_EXTENSION_NAME=" + name, "-DTORCH_API_INCLUDE_EXTENSION_H", "-D_GLIBCXX_USE_CXX11_ABI=1"]
    o_cpp, o_cu = bdir / "wrap.o", bdir / "kern.o"
    cmds = [
        ["g++", "-O3", "-std=c++17", "-fPIC", *defs, *inc, "-I/usr/local/cuda/include", "-c", str(vdir / cpp), "-o", str(o_cpp)],
        [nvcc(), *ARCH, "-O3", "-std=c++17", "-lineinfo", "--use_fast_math", "-Xcompiler", "-fPIC", "-c", str(vdir / cu),
         "-o", str(o_cu)],
    ]
    with cf.ThreadPoolExecutor(max_workers=2) as ex:
        list(ex.map(_run, cmds))
    _run([nvcc(), *ARCH, "-shared", "-o", str(out), str(o_cpp), str(o_cu), *[f for f in ld if not f.startswith("-Wl")],
          *["-Xlinker=" + f[4:] for f in ld if f.startswith("-Wl,")]])
    return out


def build_all(variants: bool = True, force: bool = False, verbose: bool = False) -> None:
    build_library(force=force, verbose=verbose)
    build_probe(force=force)
    build_trace(force=force)
    build_debug(force=force)
    if variants:
        with cf.ThreadPoolExecutor(max_workers=3) as ex:
            list(ex.map(lambda v: build_variant(v, force=force), VARIANTS))


def main(argv: list[str] | None = None) -> int:
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--no-variants", action="store_true", help="build only libgemm_b200.so")
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true", help="pass -Xptxas=-v")
    ap.add_argument("--tuning", action="store_true", help="also build the kernel variants only tuning sweeps use")
    ap.add_argument("--trace", action="store_true", help="build only the stage-timeline variant of the library (profiling/)")
    ap.add_argument("--debug", action="store_true", help="build only the bounds-checking variant of the library (profiling/)")
    a = ap.parse_args(argv)
    if a.trace:
        print(build_trace(force=True))
        return 0
    if a.debug:
        print(build_debug(force=True))
        return 0
    if a.tuning:
        TUNING.append("-DGEMM_B200_TUNING")
        a.force = True
    build_all(variants=not a.no_variants, force=a.force, verbose=a.verbose)
    print(LIB)
    return 0


if __name__ == "__main__":
    sys.exit(main())
