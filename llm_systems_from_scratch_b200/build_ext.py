"""In-tree build of the sm_100a kernel library with plain nvcc.

The kernels expose a C ABI (raw device pointers + a CUDA stream) and are loaded with
ctypes, so no PyTorch headers are needed and a full rebuild takes seconds.  The shared
object is written next to this file (``_b200_kernels.so``): it is git-ignored but
travels with the source tree to the GPU machine.

Usage:  python -m llm_systems_from_scratch_b200.build_ext [--force] [--verbose]
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
CSRC = PKG_DIR / "csrc"
BUILD_DIR = PKG_DIR / "csrc" / "build"
LIB_PATH = PKG_DIR / "_b200_kernels.so"
HOST_SRC = CSRC / "host" / "host_runtime.cpp"
HOST_LIB_PATH = PKG_DIR / "_b200_host.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
    "-Xptxas", "-v",
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found; set NVCC or add it to PATH")


def sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu"))


def _digest(paths: list[Path]) -> str:
    h = hashlib.sha256()
    for p in sorted(paths):
        h.update(p.name.encode())
        h.update(p.read_bytes())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def needs_build() -> bool:
    stamp = BUILD_DIR / "stamp.txt"
    if not LIB_PATH.exists() or not stamp.exists():
        return True
    deps = sources() + sorted(CSRC.glob("*.cuh")) + sorted(CSRC.glob("*.h"))
    return stamp.read_text().strip() != _digest(deps)


def build_host(force: bool = False) -> Path | None:
    """Compile the host-side runtime (loader gather, KV page allocator) with g++; returns None without a compiler."""
    if not HOST_SRC.exists():
        return None
    stamp = BUILD_DIR / "host_stamp.txt"
    digest = hashlib.sha256(HOST_SRC.read_bytes()).hexdigest()
    if not force and HOST_LIB_PATH.exists() and stamp.exists() and stamp.read_text().strip() == digest:
        return HOST_LIB_PATH
    cxx = os.environ.get("CXX") or shutil.which("g++") or shutil.which("c++")
    if not cxx:
        return None
    BUILD_DIR.mkdir(parents=True, exist_ok=True)
    tmp = HOST_LIB_PATH.with_suffix(".so.tmp")
    proc = subprocess.run([cxx, "-O3", "-std=c++17", "-shared", "-fPIC", "-pthread", "-o", str(tmp), str(HOST_SRC)],
                          capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError(f"host runtime build failed:\n{proc.stdout}\n{proc.stderr}")
    os.replace(tmp, HOST_LIB_PATH)
    stamp.write_text(digest)
    return HOST_LIB_PATH


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile every ``csrc/*.cu`` for sm_100a and link ``_b200_kernels.so``; also builds the host runtime."""
    build_host(force)
    if not force and not needs_build():
        return LIB_PATH
    nvcc = _nvcc()
    BUILD_DIR.mkdir(parents=True, exist_ok=True)
    srcs = sources()
    if not srcs:
        raise RuntimeError(f"no CUDA sources under {CSRC}")

    def compile_one(src: Path):
        obj = BUILD_DIR / (src.stem + ".o")
        cmd = [nvcc, *NVCC_FLAGS, "-I", str(CSRC), "-c", str(src), "-o", str(obj)]
        proc = subprocess.run(cmd, capture_output=True, text=True)
        log = BUILD_DIR / (src.stem + ".ptxas.log")
        log.write_text(proc.stdout + proc.stderr)
        if proc.returncode != 0:
            raise RuntimeError(f"nvcc failed for {src.name}:\n{proc.stdout}\n{proc.stderr}")
        if verbose:
            sys.stderr.write(proc.stderr)
        return obj

    with ThreadPoolExecutor(max_workers=min(8, len(srcs))) as ex:
        objs = list(ex.map(compile_one, srcs))
    tmp = LIB_PATH.with_suffix(".so.tmp")
    link = [nvcc, "-shared", "-o", str(tmp), *map(str, objs)]
    proc = subprocess.run(link, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError(f"link failed:\n{proc.stdout}\n{proc.stderr}")
    os.replace(tmp, LIB_PATH)
    deps = srcs + sorted(CSRC.glob("*.cuh")) + sorted(CSRC.glob("*.h"))
    (BUILD_DIR / "stamp.txt").write_text(_digest(deps))
    return LIB_PATH


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="--verbose" in sys.argv)
    print(path)
