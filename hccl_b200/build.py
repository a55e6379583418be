"""Builds the native library ``hccl_b200/lib/libhccl_b200.so`` in-tree.

Every ``.cu`` file is compiled by nvcc for sm_100a only
(``-gencode arch=compute_100a,code=sm_100a -lineinfo``), every ``.cc`` file by
g++; objects are cached under ``build/obj`` and rebuilt when the source or any
header is newer.  Usage: ``python hccl_b200/build.py [--force] [--verbose] [--ptxas] [--asan] [--trace]``.

``--asan`` builds a second library, ``build/lib/libhccl_b200_asan.so``, whose host code (every ``.cc`` file: API, selector,
bootstrap, host engine, verifier) is compiled with AddressSanitizer; the CUDA objects are shared with the normal
build.  Load it with ``HCCL_B200_LIB=<path> LD_PRELOAD=$(gcc -print-file-name=libasan.so)`` (the interpreter itself
is not instrumented, so the runtime has to come first), ``ASAN_OPTIONS=detect_leaks=0``.
``--cov`` builds ``build/lib/libhccl_b200_cov.so`` with ``--coverage``; after running tests against it
(``HCCL_B200_LIB=<path>``), ``--cov-report`` prints the line coverage of every host source.
"""
from __future__ import annotations

import concurrent.futures
import os
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
CSRC = ROOT / "csrc"
OBJ = ROOT / "build" / "obj"
LIB_DIR = ROOT / "hccl_b200" / "lib"
LIB = LIB_DIR / "libhccl_b200.so"
CUDA_HOME = Path(os.environ.get("CUDA_HOME", "/usr/local/cuda"))
NVCC = str(CUDA_HOME / "bin" / "nvcc")

NVCC_FLAGS = [
    "-std=c++17", "-O3", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=default", "--expt-relaxed-constexpr",
    f"-I{CSRC / 'include'}", f"-I{CSRC}",
]
CXX_FLAGS = [
    "-std=c++17", "-O2", "-g", "-fPIC", "-Wall", "-Wno-unused-function", "-pthread",
    f"-I{CSRC / 'include'}", f"-I{CSRC}", f"-I{CUDA_HOME / 'include'}",
]


def _sources():
    cu = sorted(CSRC.rglob("*.cu"))
    cc = sorted(CSRC.rglob("*.cc"))
    return cu, cc


def _newest_header() -> float:
    t = 0.0
    for pat in ("*.h", "*.cuh", "*.hpp"):
        for h in CSRC.rglob(pat):
            t = max(t, h.stat().st_mtime)
    return t


ASAN_FLAGS = ["-fsanitize=address", "-fno-omit-frame-pointer", "-O1"]
OBJ_ASAN = ROOT / "build" / "obj_asan"
LIB_ASAN = ROOT / "build" / "lib" / "libhccl_b200_asan.so"      # beside the objects: a test artefact, not shipped


def _compile(src: Path, verbose: bool, extra_flags=(), obj_dir: Path = None, cxx_extra=()):
    rel = src.relative_to(CSRC)
    obj = (obj_dir or OBJ) / (str(rel).replace("/", "__") + ".o")
    if src.suffix == ".cu":
        cmd = [NVCC, *NVCC_FLAGS, *extra_flags, "-c", str(src), "-o", str(obj)]
    else:
        cmd = ["g++", *CXX_FLAGS, *cxx_extra, "-c", str(src), "-o", str(obj)]
    if verbose:
        print(" ".join(cmd), flush=True)
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"compiling {rel} failed:\n{r.stdout}\n{r.stderr}")
    if verbose and r.stderr.strip():
        print(r.stderr)
    return obj


def build(force: bool = False, verbose: bool = False, ptxas_verbose: bool = False) -> Path:
    OBJ.mkdir(parents=True, exist_ok=True)
    LIB_DIR.mkdir(parents=True, exist_ok=True)
    cu, cc = _sources()
    hdr_time = _newest_header()
    todo, objs = [], []
    for src in cu + cc:
        rel = src.relative_to(CSRC)
        obj = OBJ / (str(rel).replace("/", "__") + ".o")
        objs.append(obj)
        if force or not obj.exists() or obj.stat().st_mtime < max(src.stat().st_mtime, hdr_time):
            todo.append(src)
    extra = ("-Xptxas", "-v") if ptxas_verbose else ()
    if todo:
        workers = min(len(todo), max(1, (os.cpu_count() or 4)))
        with concurrent.futures.ThreadPoolExecutor(workers) as ex:
            list(ex.map(lambda s: _compile(s, verbose or ptxas_verbose, extra), todo))
    if todo or not LIB.exists():
        cmd = [NVCC, "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", str(LIB), *map(str, objs), "-Xcompiler", "-pthread", "-ldl", "-lrt"]
        if verbose:
            print(" ".join(cmd), flush=True)
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"linking failed:\n{r.stdout}\n{r.stderr}")
    return LIB


def _build_variant(obj_dir: Path, lib: Path, cxx_extra, link_extra, verbose: bool) -> Path:
    """A variant of the library whose host objects are compiled with extra flags; the CUDA objects are shared."""
    build(verbose=verbose)
    obj_dir.mkdir(parents=True, exist_ok=True)
    lib.parent.mkdir(parents=True, exist_ok=True)
    cu, cc = _sources()
    hdr_time = _newest_header()
    todo, objs = [], []
    for src in cu:
        objs.append(OBJ / (str(src.relative_to(CSRC)).replace("/", "__") + ".o"))
    for src in cc:
        obj = obj_dir / (str(src.relative_to(CSRC)).replace("/", "__") + ".o")
        objs.append(obj)
        if not obj.exists() or obj.stat().st_mtime < max(src.stat().st_mtime, hdr_time):
            todo.append(src)
    if todo:
        with concurrent.futures.ThreadPoolExecutor(min(len(todo), max(1, (os.cpu_count() or 4)))) as ex:
            list(ex.map(lambda s: _compile(s, verbose, (), obj_dir, cxx_extra), todo))
    if todo or not lib.exists():
        cmd = [NVCC, "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", str(lib), *map(str, objs), "-Xcompiler", "-pthread",
               *link_extra, "-ldl", "-lrt"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"linking {lib.name} failed:\n{r.stdout}\n{r.stderr}")
    return lib


def build_asan(verbose: bool = False) -> Path:
    """The AddressSanitizer variant: instrumented host objects + the CUDA objects of the normal build."""
    return _build_variant(OBJ_ASAN, LIB_ASAN, ASAN_FLAGS, ["-Xcompiler", "-fsanitize=address"], verbose)


OBJ_TRACE = ROOT / "build" / "obj_trace"
LIB_TRACE = ROOT / "build" / "lib" / "libhccl_b200_trace.so"


def build_trace(verbose: bool = False) -> Path:
    """The timeline variant: the fused matmul kernels compiled with -DHCCL_MC2_TRACE (every role of every CTA writes
    where its time went; `HCCL_MC2_TRACE_FILE=<prefix>` dumps launches `HCCL_MC2_TRACE_FROM`..+2 as JSON lines), all
    other objects shared with the normal build.  Load it with `HCCL_B200_LIB=<path>`; a tool for performance work,
    not for timing (the trace costs a few per cent)."""
    build(verbose=verbose)
    OBJ_TRACE.mkdir(parents=True, exist_ok=True)
    LIB_TRACE.parent.mkdir(parents=True, exist_ok=True)
    cu, cc = _sources()
    objs = []
    for src in cu + cc:
        if src.name == "mc2_launch.cu":
            objs.append(_compile(src, verbose, ("-DHCCL_MC2_TRACE",), OBJ_TRACE))
        else:
            objs.append(OBJ / (str(src.relative_to(CSRC)).replace("/", "__") + ".o"))
    cmd = [NVCC, "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", str(LIB_TRACE), *map(str, objs), "-Xcompiler", "-pthread", "-ldl", "-lrt"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"linking {LIB_TRACE.name} failed:\n{r.stdout}\n{r.stderr}")
    return LIB_TRACE


OBJ_COV = ROOT / "build" / "obj_cov"
LIB_COV = ROOT / "build" / "lib" / "libhccl_b200_cov.so"


def build_cov(verbose: bool = False) -> Path:
    """The coverage variant (gcc --coverage): run tests with HCCL_B200_LIB pointing at it, then `--cov-report`."""
    return _build_variant(OBJ_COV, LIB_COV, ["--coverage", "-O0"], ["-Xcompiler", "--coverage"], verbose)


def cov_report() -> str:
    """Line coverage of the host sources from the counters the coverage build has written so far (gcov)."""
    rows, total_lines, total_hit = [], 0, 0
    for gcda in sorted(OBJ_COV.glob("*.gcda")):
        r = subprocess.run(["gcov", "-n", "-o", str(OBJ_COV), str(gcda)], capture_output=True, text=True, cwd=OBJ_COV)
        name, own = None, False
        for line in r.stdout.splitlines():
            if line.startswith("File '"):
                name = line[6:-1]
                own = name.startswith(str(CSRC)) and name.endswith(".cc")
            elif own and line.startswith("Lines executed:"):
                pct, of = line[len("Lines executed:"):].split("% of ")
                n = int(of)
                hit = round(float(pct) * n / 100.0)
                rows.append((str(Path(name).relative_to(CSRC)), hit, n))
                total_lines += n
                total_hit += hit
                own = False
    out = [f"{100.0 * h / n:6.1f} %  {h:5d} / {n:5d}  {f}" for f, h, n in sorted(rows)]
    out.append(f"{100.0 * total_hit / max(1, total_lines):6.1f} %  {total_hit:5d} / {total_lines:5d}  all host sources")
    return "\n".join(out)


if __name__ == "__main__":
    if "--asan" in sys.argv:
        print(build_asan(verbose="--verbose" in sys.argv))
        sys.exit(0)
    if "--trace" in sys.argv:
        print(build_trace(verbose="--verbose" in sys.argv))
        sys.exit(0)
    if "--cov" in sys.argv:
        print(build_cov(verbose="--verbose" in sys.argv))
        sys.exit(0)
    if "--cov-report" in sys.argv:
        print(cov_report())
        sys.exit(0)
    lib = build(force="--force" in sys.argv, verbose="--verbose" in sys.argv, ptxas_verbose="--ptxas" in sys.argv)
    print(lib)
