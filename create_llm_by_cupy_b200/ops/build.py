"""In-tree build of the native library (``libb200llm.so``) with nvcc for sm_100a.

The library exposes a plain ``extern "C"`` surface that is loaded with ctypes, so it needs
neither the torch headers nor a Python ABI: a full rebuild is a few nvcc invocations run in
parallel. nvcc cross-compiles, so the build also runs on a machine without a GPU.

    python -m create_llm_by_cupy_b200.ops.build [--force] [--verbose]
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

CSRC = Path(__file__).resolve().parent / "csrc"
OUT_DIR = Path(__file__).resolve().parent

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
    "--expt-relaxed-constexpr",
]
# Approximate division / exp / rsqrt only where the arithmetic feeds bf16 tensor-core operands anyway (the
# attention and GEMM units). The optimizer, the normalisation and the loss kernels keep IEEE division and
# square roots: their results go into fp32 state.
FAST_MATH_PREFIXES = ("flash_", "gemm_")
# ``B200_BOUNDS_CHECK=1``: debug build in which the kernels that take indices or offsets from their
# arguments check them (and report through the status word instead of touching memory) - the stand-in for
# a memory checker. Objects of the two builds are kept apart by the flag's part in the digest.
BOUNDS_CHECK = os.environ.get("B200_BOUNDS_CHECK") == "1"
LIB_NAME = "libb200llm_dbg.so" if BOUNDS_CHECK else "libb200llm.so"
OBJ_DIR_NAME = "build_dbg" if BOUNDS_CHECK else "build"


def flags_for(src: Path) -> list[str]:
    fl = list(NVCC_FLAGS)
    if src.name.startswith(FAST_MATH_PREFIXES):
        fl.append("--use_fast_math")
    if BOUNDS_CHECK:
        fl.append("-DB200_BOUNDS_CHECK=1")
    return fl


def _nvcc() -> str:
    cand = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(cand):
        raise RuntimeError("nvcc not found: the native library cannot be built")
    return cand


def sources() -> list[Path]:
    return sorted(list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cpp")))


def _digest(src: Path) -> str:
    h = hashlib.sha1()
    h.update(src.read_bytes())
    for hdr in sorted(CSRC.glob("*.cuh")) + sorted(CSRC.glob("*.h")):
        h.update(hdr.read_bytes())
    h.update(" ".join(flags_for(src)).encode())
    return h.hexdigest()


def lib_path() -> Path:
    return OUT_DIR / LIB_NAME


def source_digest() -> str:
    """One digest over every source, header and the compiler flags: names the code a library was built from."""
    h = hashlib.sha1()
    for src in sources():
        h.update(_digest(src).encode())
    return h.hexdigest()


def is_current() -> bool:
    """True when the library exists and every object's stamp matches its source as it is now."""
    if not lib_path().exists():
        return False
    obj_dir = OUT_DIR / OBJ_DIR_NAME
    for src in sources():
        stamp = obj_dir / (src.stem + ".sha1")
        if not stamp.exists() or stamp.read_text() != _digest(src):
            return False
    return True


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile every source under ``csrc/`` that changed and link ``libb200llm.so``. Processes that
    build at the same time (one per GPU at start-up) take turns on a lock file; the second one then finds
    everything up to date."""
    nvcc = _nvcc()
    obj_dir = OUT_DIR / OBJ_DIR_NAME
    obj_dir.mkdir(exist_ok=True)
    import fcntl
    with open(obj_dir / ".lock", "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        try:
            return _build_locked(nvcc, obj_dir, force, verbose)
        finally:
            fcntl.flock(lock, fcntl.LOCK_UN)


def _build_locked(nvcc: str, obj_dir: Path, force: bool, verbose: bool) -> Path:
    jobs = []
    objs = []
    for src in sources():
        obj = obj_dir / (src.stem + ".o")
        stamp = obj_dir / (src.stem + ".sha1")
        objs.append(obj)
        dig = _digest(src)
        if not force and obj.exists() and stamp.exists() and stamp.read_text() == dig:
            continue
        cmd = [nvcc, *flags_for(src), "-I", str(CSRC), "-c", str(src), "-o", str(obj)]
        if src.suffix == ".cpp":
            cmd = [nvcc, "-O3", "-std=c++17", "-Xcompiler", "-fPIC,-fopenmp,-march=x86-64-v3,-fvisibility=hidden",
                   "-I", str(CSRC), "-c", str(src), "-o", str(obj)]
        if verbose and src.suffix == ".cu":
            cmd += ["-Xptxas", "-v"]
        jobs.append((cmd, stamp, dig, src))

    def run(job):
        cmd, stamp, dig, src = job
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed for {src.name}:\n{r.stdout}\n{r.stderr}")
        if verbose:
            print(r.stderr, file=sys.stderr)
        stamp.write_text(dig)
        return src.name

    if jobs:
        with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            for name in ex.map(run, jobs):
                if verbose:
                    print(f"[build] compiled {name}", file=sys.stderr)
    out = lib_path()
    if jobs or not out.exists():
        tmp = out.with_suffix(".so.tmp")
        cmd = [nvcc, "-shared", "-o", str(tmp), *map(str, objs), "-Xcompiler", "-fopenmp"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
        os.replace(tmp, out)
    return out


if __name__ == "__main__":
    p = build(force="--force" in sys.argv, verbose="--verbose" in sys.argv)
    print(p)
