"""In-tree build of the C++ device runtime (`nkipy_b200/spike/_spike*.so`).

Plain g++ against pybind11 and the CUDA headers; the driver library itself is loaded
with dlopen at run time, so the module builds and imports without a GPU.
"""

from __future__ import annotations

import hashlib
import os
import subprocess
import sys
import sysconfig
from pathlib import Path

ROOT = Path(__file__).resolve().parents[2]
SRC_DIR = ROOT / "csrc" / "runtime"
OUT_DIR = ROOT / "nkipy_b200" / "spike"
BUILD_DIR = ROOT / "build" / "runtime"


def module_path() -> Path:
    return OUT_DIR / f"_spike{sysconfig.get_config_var('EXT_SUFFIX')}"


def build(force: bool = False) -> Path:
    import pybind11

    srcs = sorted(SRC_DIR.glob("*.cpp"))
    deps = srcs + sorted(SRC_DIR.glob("*.h")) + [ROOT / "csrc" / "kernels" / "gemm_args.h"]
    h = hashlib.sha256()
    for d in deps:
        h.update(d.read_bytes())
    stamp = h.hexdigest()[:16]
    BUILD_DIR.mkdir(parents=True, exist_ok=True)
    stamp_file = BUILD_DIR / "stamp"
    out = module_path()

    def fresh() -> bool:
        return out.exists() and stamp_file.exists() and stamp_file.read_text() == stamp

    if not force and fresh():
        return out
    import fcntl

    # several rank processes may get here at once: one builds, the others wait and find it done; the module is
    # linked under a temporary name and moved into place, so nobody ever maps a half-written file
    with open(BUILD_DIR / "lock", "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        try:
            if not force and fresh():
                return out
            cuda_inc = os.environ.get("CUDA_HOME", "/usr/local/cuda") + "/include"
            tmp = out.with_name(out.name + f".tmp{os.getpid()}")
            cmd = ["g++", "-O2", "-std=c++17", "-shared", "-fPIC", "-fvisibility=hidden", "-Wall",
                   f"-I{pybind11.get_include()}", f"-I{sysconfig.get_paths()['include']}", f"-I{cuda_inc}",
                   *[str(s) for s in srcs], "-o", str(tmp), "-ldl", "-lpthread"]
            res = subprocess.run(cmd, capture_output=True, text=True)
            if res.returncode != 0:
                if tmp.exists():
                    tmp.unlink()
                raise RuntimeError(f"building the device runtime failed:\n{' '.join(cmd)}\n{res.stdout}\n{res.stderr}")
            os.replace(tmp, out)
            stamp_file.write_text(stamp)
        finally:
            fcntl.flock(lock, fcntl.LOCK_UN)
    return out


def _source_digest() -> str:
    h = hashlib.sha256()
    for d in sorted(SRC_DIR.glob("*.cpp")) + sorted(SRC_DIR.glob("*.h")) + [ROOT / "csrc" / "kernels" / "gemm_args.h"]:
        h.update(d.read_bytes())
    return h.hexdigest()[:16]


def build_sanitized(out_dir=None) -> Path:
    """The runtime module built with AddressSanitizer and UndefinedBehaviorSanitizer, for tests that drive it on the
    host against a stand-in driver library.  A process that imports it must preload the sanitizer runtime
    (`sanitizer_preload()`), because the interpreter itself is not instrumented."""
    import pybind11

    out_dir = Path(out_dir) if out_dir is not None else BUILD_DIR / "sanitized"      # kept between runs: the build takes a while
    out_dir.mkdir(parents=True, exist_ok=True)
    out = out_dir / module_path().name
    stamp, stamp_file = _source_digest(), out_dir / "stamp"
    if out.exists() and stamp_file.exists() and stamp_file.read_text() == stamp:
        return out
    cuda_inc = os.environ.get("CUDA_HOME", "/usr/local/cuda") + "/include"
    cmd = ["g++", "-O1", "-g", "-std=c++17", "-shared", "-fPIC", "-fvisibility=hidden", "-Wall",
           "-fsanitize=address,undefined", "-fno-sanitize-recover=all", "-fno-omit-frame-pointer",
           f"-I{pybind11.get_include()}", f"-I{sysconfig.get_paths()['include']}", f"-I{cuda_inc}",
           *[str(s) for s in sorted(SRC_DIR.glob("*.cpp"))], "-o", str(out), "-ldl", "-lpthread"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"building the sanitized runtime failed:\n{' '.join(cmd)}\n{res.stdout}\n{res.stderr}")
    stamp_file.write_text(stamp)
    return out


def sanitizer_preload() -> str:
    """Value for LD_PRELOAD: the shared AddressSanitizer runtime of the host compiler, followed by the C++ runtime
    library (the interpreter does not link it, and the sanitizer must find `__cxa_throw` when it starts)."""
    paths = []
    for lib in ("libasan.so", "libstdc++.so.6"):
        res = subprocess.run(["g++", f"-print-file-name={lib}"], capture_output=True, text=True)
        path = res.stdout.strip()
        if not os.path.isabs(path):
            return ""
        paths.append(os.path.realpath(path))
    return " ".join(paths)


if __name__ == "__main__":
    print(build(force="--force" in sys.argv))
