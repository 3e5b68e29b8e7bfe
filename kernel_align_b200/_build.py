"""In-tree native build: nvcc for the sm_100a kernels, g++ for the CPU oracle library.

Both libraries are plain shared objects with ``extern "C"`` entry points, loaded through
``ctypes``; they sit next to the package so that a built tree can be copied to a GPU host
as is. A content hash of the sources and flags decides whether a rebuild is needed.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
CSRC = ROOT / "csrc"
LIB_DIR = Path(__file__).resolve().parent / "_lib"
OBJ_DIR = ROOT / "build" / "obj"

CUDA_LIB = LIB_DIR / "libka_sm100.so"
CPU_LIB = LIB_DIR / "libka_cpu.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
    "--expt-relaxed-constexpr",
    "-diag-suppress", "177",
]
CXX_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-ffp-contract=off", "-fno-fast-math", "-pthread"]


def _nvcc() -> str | None:
    cand = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    return cand if os.path.exists(cand) else None


def _digest(files: list[Path], flags: list[str]) -> str:
    h = hashlib.sha256()
    h.update(" ".join(flags).encode())
    for f in sorted(files):
        h.update(str(f.relative_to(ROOT)).encode())
        h.update(f.read_bytes())
    return h.hexdigest()


def _run(cmd: list[str]) -> None:
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        sys.stderr.write(" ".join(cmd) + "\n" + r.stdout + r.stderr)
        raise RuntimeError(f"native build failed: {' '.join(cmd[:3])} ...")


def _stamp_ok(lib: Path, digest: str) -> bool:
    stamp = lib.with_suffix(".hash")
    return lib.exists() and stamp.exists() and stamp.read_text().strip() == digest


def build_cuda(force: bool = False, verbose: bool = False) -> Path | None:
    """Compile every ``csrc/sm100/*.cu`` for sm_100a and link ``libka_sm100.so``."""
    nvcc = _nvcc()
    srcs = sorted((CSRC / "sm100").glob("*.cu"))
    if not srcs:      # an installed wheel carries the built library, not the sources
        return CUDA_LIB if CUDA_LIB.exists() else None
    deps = srcs + sorted((CSRC / "sm100").rglob("*.cuh")) + sorted((CSRC / "sm100").rglob("*.h"))
    digest = _digest(deps, NVCC_FLAGS)
    if not force and _stamp_ok(CUDA_LIB, digest):
        return CUDA_LIB
    if nvcc is None:
        return CUDA_LIB if CUDA_LIB.exists() else None
    LIB_DIR.mkdir(parents=True, exist_ok=True)
    OBJ_DIR.mkdir(parents=True, exist_ok=True)
    extra = ["-Xptxas", "-v"] if verbose else []

    def one(src: Path) -> Path:
        obj = OBJ_DIR / (src.stem + ".o")
        _run([nvcc, *NVCC_FLAGS, *extra, "-I", str(CSRC / "sm100"), "-c", str(src), "-o", str(obj)])
        return obj

    with ThreadPoolExecutor(max_workers=min(8, max(1, len(srcs)))) as ex:
        objs = list(ex.map(one, srcs))
    _run([nvcc, "-shared", "-o", str(CUDA_LIB), *[str(o) for o in objs], "-cudart", "static"])
    CUDA_LIB.with_suffix(".hash").write_text(digest)
    return CUDA_LIB


def build_cpu(force: bool = False) -> Path | None:
    """Compile ``csrc/cpu/*.cpp`` into ``libka_cpu.so`` (the CPU oracle and CPU code path)."""
    srcs = sorted((CSRC / "cpu").glob("*.cpp"))
    if not srcs:
        return CPU_LIB if CPU_LIB.exists() else None
    deps = srcs + sorted((CSRC / "cpu").rglob("*.h"))
    digest = _digest(deps, CXX_FLAGS)
    if not force and _stamp_ok(CPU_LIB, digest):
        return CPU_LIB
    cxx = shutil.which("g++")
    if cxx is None:
        return CPU_LIB if CPU_LIB.exists() else None
    LIB_DIR.mkdir(parents=True, exist_ok=True)
    _run([cxx, *CXX_FLAGS, "-shared", "-o", str(CPU_LIB), *[str(s) for s in srcs]])
    CPU_LIB.with_suffix(".hash").write_text(digest)
    return CPU_LIB


def build_cpu_sanitized(force: bool = False) -> Path | None:
    """The CPU library once more with AddressSanitizer and UndefinedBehaviorSanitizer
    (``libka_cpu_asan.so``): the sanitizer tier of the tests loads it in a child process that
    preloads the sanitizer runtime. Not used by the package itself."""
    srcs = sorted((CSRC / "cpu").glob("*.cpp"))
    cxx = shutil.which("g++")
    if not srcs or cxx is None:
        return None
    flags = [f for f in CXX_FLAGS if not f.startswith("-O")] + ["-O1", "-g", "-fno-omit-frame-pointer",
                                                                 "-fsanitize=address,undefined",
                                                                 "-fno-sanitize-recover=undefined"]
    deps = srcs + sorted((CSRC / "cpu").rglob("*.h"))
    digest = _digest(deps, flags)
    lib = LIB_DIR / "libka_cpu_asan.so"
    if not force and _stamp_ok(lib, digest):
        return lib
    LIB_DIR.mkdir(parents=True, exist_ok=True)
    _run([cxx, *flags, "-shared", "-o", str(lib), *[str(s) for s in srcs]])
    lib.with_suffix(".hash").write_text(digest)
    return lib


def sanitizer_runtime() -> str | None:
    """Path of the AddressSanitizer runtime to preload, or None without g++."""
    cxx = shutil.which("g++")
    if cxx is None:
        return None
    out = subprocess.run([cxx, "-print-file-name=libasan.so"], capture_output=True, text=True).stdout.strip()
    return out if out and os.path.exists(out) else None


def build_all(force: bool = False, verbose: bool = False) -> None:
    build_cpu(force)
    build_cuda(force, verbose)


if __name__ == "__main__":
    build_all(force="--force" in sys.argv, verbose="-v" in sys.argv)
    print("built:", [str(p) for p in (CPU_LIB, CUDA_LIB) if p.exists()])
