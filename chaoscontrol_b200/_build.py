"""In-tree native build: nvcc for the sm_100a kernel library, g++ for the CPU
control plane.  Both produce shared objects under ``chaoscontrol_b200/lib``
that the Python layer binds with ctypes, so no libtorch headers are compiled
and a full rebuild takes seconds.

The reference builds four torch C++ extensions through setup.py hooks
(setup.py:64-85 in the reference tree); here the kernels are plain
``extern "C"`` launchers and the build is two compiler invocations per file.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
NATIVE = PKG / "native"
LIBDIR = PKG / "lib"
OBJDIR = LIBDIR / "obj"

CUDA_LIB = LIBDIR / "libccb200.so"
CTRL_LIB = LIBDIR / "libccb200_ctrl.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "--expt-relaxed-constexpr",
    "-Xcompiler", "-fPIC",
    "-Xptxas", "-v",
]
CXX_FLAGS = ["-O3", "-std=c++17", "-fPIC", "-Wall", "-pthread"]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise RuntimeError("nvcc not found: cannot build the sm_100a kernel library")


def _digest(path: Path, extra: list[Path], flags: list[str]) -> str:
    h = hashlib.sha256()
    h.update(" ".join(flags).encode())
    for p in [path, *extra]:
        h.update(p.read_bytes())
    return h.hexdigest()


def _compile_one(compiler: list[str], src: Path, headers: list[Path], flags: list[str],
                 verbose: bool) -> Path:
    OBJDIR.mkdir(parents=True, exist_ok=True)
    obj = OBJDIR / (src.name + ".o")
    stamp = OBJDIR / (src.name + ".sha")
    dig = _digest(src, headers, flags)
    if obj.exists() and stamp.exists() and stamp.read_text() == dig:
        return obj
    cmd = [*compiler, *flags, "-I", str(src.parent), "-c", str(src), "-o", str(obj)]
    res = subprocess.run(cmd, capture_output=True, text=True)
    log = OBJDIR / (src.name + ".log")
    log.write_text(res.stdout + res.stderr)
    if res.returncode != 0:
        raise RuntimeError(f"compile failed: {' '.join(cmd)}\n{res.stdout}\n{res.stderr}")
    if verbose:
        for line in (res.stdout + res.stderr).splitlines():
            if "registers" in line or "spill" in line and "0 bytes spill" not in line:
                print(f"[{src.name}] {line.strip()}")
    stamp.write_text(dig)
    return obj


def build_cuda(verbose: bool = False) -> Path:
    """Compile every ``csrc/*.cu`` for sm_100a and link ``libccb200.so``."""
    nvcc = _nvcc()
    srcs = sorted(CSRC.glob("*.cu"))
    headers = sorted(CSRC.glob("*.h")) + sorted(CSRC.glob("*.cuh"))
    with ThreadPoolExecutor(max_workers=min(8, len(srcs) or 1)) as ex:
        objs = list(ex.map(lambda s: _compile_one([nvcc], s, headers, NVCC_FLAGS, verbose), srcs))
    newest = max((o.stat().st_mtime for o in objs), default=0.0)
    if not CUDA_LIB.exists() or CUDA_LIB.stat().st_mtime < newest:
        cmd = [nvcc, "-shared", "-o", str(CUDA_LIB), *map(str, objs), "-lcudart"]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"link failed: {res.stdout}\n{res.stderr}")
    return CUDA_LIB


def build_ctrl(verbose: bool = False) -> Path:
    """Compile the CPU control plane (``native/*.cpp``) into ``libccb200_ctrl.so``."""
    cxx = os.environ.get("CXX") or shutil.which("g++") or "g++"
    srcs = sorted(p for p in NATIVE.glob("*.cpp") if p.name != "selftest.cpp")   # the stress driver has a main()
    if not srcs:
        return CTRL_LIB
    headers = sorted(NATIVE.glob("*.h"))
    with ThreadPoolExecutor(max_workers=min(8, len(srcs))) as ex:
        objs = list(ex.map(lambda s: _compile_one([cxx], s, headers, CXX_FLAGS, verbose), srcs))
    newest = max((o.stat().st_mtime for o in objs), default=0.0)
    if not CTRL_LIB.exists() or CTRL_LIB.stat().st_mtime < newest:
        cmd = [cxx, "-shared", "-o", str(CTRL_LIB), *map(str, objs), "-lrt", "-pthread"]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"link failed: {res.stdout}\n{res.stderr}")
    return CTRL_LIB


SANITIZERS = ("thread", "address")


def build_and_run_selftest(sanitize: str, timeout: float = 300.0) -> tuple[int, str]:
    """Compile ``native/selftest.cpp`` with the ring, shared-memory and pad-protocol sources under
    ``-fsanitize=<thread|address>`` into ``lib/ccb200_ctrl_selftest_<sanitizer>`` and run it.
    Returns ``(exit code, combined output)``; 0 means every check held and the sanitizer stayed quiet,
    127 that the compiler has no runtime library for that sanitizer on this machine.  ``sanitize="none"``
    builds and runs the same driver without instrumentation (the functional half of the check)."""
    if sanitize not in SANITIZERS + ("none",):
        raise ValueError(f"sanitize must be one of {SANITIZERS + ('none',)}, got {sanitize!r}")
    # the sanitizer runtimes ship with the distribution's compiler, which need not be $CXX or the first
    # g++ on PATH: try each candidate until one links
    cands = [os.environ.get("CCB_SANITIZE_CXX"), "/usr/bin/g++-13", "/usr/bin/x86_64-linux-gnu-g++-13", "/usr/bin/g++",
             os.environ.get("CXX"), shutil.which("g++")]
    cands = [c for i, c in enumerate(cands) if c and Path(c).exists() and c not in cands[:i]] or ["g++"]
    LIBDIR.mkdir(parents=True, exist_ok=True)
    exe = LIBDIR / f"ccb200_ctrl_selftest_{sanitize}"
    srcs = [NATIVE / n for n in ("selftest.cpp", "ring.cpp", "pad_protocol.cpp")]
    san = [] if sanitize == "none" else [f"-fsanitize={sanitize}"]
    missing = []
    for cxx in cands:
        cmd = [cxx, "-std=c++17", "-O1", "-g", "-fno-omit-frame-pointer", *san, "-pthread",
               "-I", str(NATIVE), *map(str, srcs), "-o", str(exe), "-lrt"]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode == 0:
            break
        if "cannot find -ltsan" in res.stderr or "cannot find -lasan" in res.stderr or "preinit.o" in res.stderr:
            missing.append(cxx)
            continue
        return res.returncode, f"compile failed: {' '.join(cmd)}\n{res.stdout}\n{res.stderr}"
    else:
        return 127, f"no sanitizer runtime for -fsanitize={sanitize} with any of {missing}"
    env = dict(os.environ)
    env.setdefault("TSAN_OPTIONS", "halt_on_error=1 exitcode=66 second_deadlock_stack=1")
    env.setdefault("ASAN_OPTIONS", "detect_leaks=1 exitcode=66")
    run = [str(exe)]
    if sanitize == "thread" and shutil.which("setarch"):
        run = ["setarch", "-R", *run]          # ThreadSanitizer's shadow layout wants ASLR off on recent kernels
    out = subprocess.run(run, capture_output=True, text=True, timeout=timeout, env=env)
    return out.returncode, out.stdout + out.stderr


def build_all(verbose: bool = False) -> dict[str, str]:
    LIBDIR.mkdir(parents=True, exist_ok=True)
    return {"cuda": str(build_cuda(verbose)), "ctrl": str(build_ctrl(verbose))}


if __name__ == "__main__":
    if "--sanitize" in sys.argv:
        which = sys.argv[sys.argv.index("--sanitize") + 1]
        rc, text = build_and_run_selftest(which)
        print(text.strip())
        print(f"selftest under -fsanitize={which}: exit code {rc}")
        sys.exit(rc)
    out = build_all(verbose="-v" in sys.argv)
    for k, v in out.items():
        print(f"{k}: {v}")
