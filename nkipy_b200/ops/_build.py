"""In-tree build of the sm_100a kernel library.

`build()` compiles every ``csrc/kernels/*.cu`` with nvcc for
``compute_100a/sm_100a`` and links them into
``nkipy_b200/ops/libnkipy_b200_kernels.so`` next to this file.  The library
exposes a C ABI (see ``csrc/kernels/api.h``) that ``_lib.py`` binds with ctypes,
so no torch C++ headers are needed and a file compiles in seconds.  nvcc
cross-compiles without a GPU; objects are cached by source hash under
``build/kernels``.
"""

from __future__ import annotations

import contextlib
import fcntl
import hashlib
import os
import shutil
import subprocess
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

ROOT = Path(__file__).resolve().parents[2]
SRC_DIR = ROOT / "csrc" / "kernels"
OBJ_DIR = ROOT / "build" / "kernels"
LIB_PATH = Path(__file__).resolve().parent / "libnkipy_b200_kernels.so"
# digest of every source, header and flag the library was built from; `_lib.lib()` refuses to load a
# library whose stamp does not match the sources (the ctypes signatures are declared from the sources,
# so a stale binary would receive shifted arguments)
STAMP_PATH = LIB_PATH.with_name(LIB_PATH.name + ".stamp")

NVCC_FLAGS = [
    "-std=c++17",
    "-gencode",
    "arch=compute_100a,code=sm_100a",
    "-lineinfo",
    "-O3",
    "--use_fast_math",
    "-Xcompiler",
    "-fPIC",
]
# fast-math turns exp2f / division into their approximate forms, which is what the
# GEMM epilogue and the attention softmax want; the normalisation and sampling
# files keep IEEE division and sqrt.
NO_FAST_MATH = {"sampling.cu", "elementwise.cu", "decode_layer.cu"}


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found; set NVCC or install the CUDA toolkit")


def _digest(path: Path, flags) -> str:
    h = hashlib.sha256()
    h.update(" ".join(flags).encode())
    h.update(path.read_bytes())
    for dep in sorted(SRC_DIR.glob("*.cuh")) + sorted(SRC_DIR.glob("*.h")):
        h.update(dep.read_bytes())
    return h.hexdigest()[:16]


def sources():
    return sorted(SRC_DIR.glob("*.cu"))


def source_digest() -> str:
    """One digest over the flags and all kernel sources and headers."""
    h = hashlib.sha256()
    h.update(" ".join(NVCC_FLAGS).encode())
    h.update(",".join(sorted(NO_FAST_MATH)).encode())
    for f in sources() + sorted(SRC_DIR.glob("*.cuh")) + sorted(SRC_DIR.glob("*.h")):
        h.update(f.name.encode())
        h.update(f.read_bytes())
    return h.hexdigest()[:24]


def is_stale() -> bool:
    """True when the library is missing or was built from other sources than the ones in the tree."""
    if not LIB_PATH.exists() or not STAMP_PATH.exists():
        return True
    return STAMP_PATH.read_text().strip() != source_digest()


@contextlib.contextmanager
def _build_lock():
    """Exclusive inter-process lock: several ranks of one job may find the library stale at once."""
    OBJ_DIR.mkdir(parents=True, exist_ok=True)
    with open(OBJ_DIR / ".lock", "w") as fh:
        fcntl.flock(fh, fcntl.LOCK_EX)
        try:
            yield
        finally:
            fcntl.flock(fh, fcntl.LOCK_UN)


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile (if stale) and link the kernel library; returns its path.  Safe to call from several
    processes at once: one builds under a file lock, the others find the result up to date."""
    with _build_lock():
        if not force and not is_stale():
            return LIB_PATH
        return _build_locked(force, verbose)


def _build_locked(force: bool, verbose: bool) -> Path:
    nvcc = _nvcc()
    OBJ_DIR.mkdir(parents=True, exist_ok=True)
    digest = source_digest()
    jobs = []
    for src in sources():
        flags = [f for f in NVCC_FLAGS if not (f == "--use_fast_math" and src.name in NO_FAST_MATH)]
        obj = OBJ_DIR / f"{src.stem}.{_digest(src, flags)}.o"
        jobs.append((src, obj, flags))

    def compile_one(job):
        src, obj, flags = job
        if obj.exists() and not force:
            return None
        for old in OBJ_DIR.glob(f"{src.stem}.*.o"):
            old.unlink()
        tmp = obj.with_suffix(f".tmp{os.getpid()}.o")
        cmd = [nvcc, *flags, "-I", str(SRC_DIR), "-c", str(src), "-o", str(tmp)]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"nvcc failed for {src.name}:\n{' '.join(cmd)}\n{res.stdout}\n{res.stderr}")
        os.replace(tmp, obj)
        return res.stderr if verbose else None

    with ThreadPoolExecutor(max_workers=min(8, len(jobs) or 1)) as pool:
        rebuilt = list(pool.map(compile_one, jobs))
    objs = [str(o) for _, o, _ in jobs]
    stamp = hashlib.sha256("".join(objs).encode()).hexdigest()[:16]
    stamp_file = OBJ_DIR / "link.stamp"
    if force or not LIB_PATH.exists() or not stamp_file.exists() or stamp_file.read_text() != stamp:
        # link under a temporary name and move it into place: a process that has the old file mapped keeps it
        tmp_lib = LIB_PATH.with_name(f".{LIB_PATH.name}.tmp{os.getpid()}")
        cmd = [nvcc, "-shared", "-o", str(tmp_lib), *objs, "-gencode", "arch=compute_100a,code=sm_100a"]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"link failed:\n{' '.join(cmd)}\n{res.stdout}\n{res.stderr}")
        os.replace(tmp_lib, LIB_PATH)
        stamp_file.write_text(stamp)
    STAMP_PATH.write_text(digest)
    if verbose:
        for msg in rebuilt:
            if msg:
                print(msg)
    return LIB_PATH


if __name__ == "__main__":
    print(build(verbose=True))
