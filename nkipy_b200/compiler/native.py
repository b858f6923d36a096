"""In-tree build of the native compiler: the `_b200c` Python module and the
`nkipy-b200-opt` command-line driver (plain g++, no external dependencies)."""

from __future__ import annotations

import hashlib
import subprocess
import sys
import sysconfig
from pathlib import Path

ROOT = Path(__file__).resolve().parents[2]
SRC_DIR = ROOT / "csrc" / "compiler"
OUT_DIR = ROOT / "nkipy_b200" / "nkigen"
BUILD_DIR = ROOT / "build" / "compiler"


def module_path() -> Path:
    return OUT_DIR / f"_b200c{sysconfig.get_config_var('EXT_SUFFIX')}"


def opt_path() -> Path:
    return OUT_DIR / "nkipy-b200-opt"


def build(force: bool = False):
    import pybind11

    deps = sorted(SRC_DIR.glob("*.cpp")) + sorted(SRC_DIR.glob("*.h")) + [ROOT / "csrc" / "runtime" / "json.h"]
    h = hashlib.sha256()
    for d in deps:
        h.update(d.read_bytes())
    stamp = h.hexdigest()[:16]
    BUILD_DIR.mkdir(parents=True, exist_ok=True)
    stamp_file = BUILD_DIR / "stamp"
    def fresh() -> bool:
        return (module_path().exists() and opt_path().exists() and stamp_file.exists()
                and stamp_file.read_text() == stamp)

    if not force and fresh():
        return module_path(), opt_path()
    import fcntl
    import os

    lib = [str(SRC_DIR / "ir.cpp"), str(SRC_DIR / "passes.cpp")]
    common = ["g++", "-O2", "-std=c++17", "-Wall", "-fPIC"]
    # one process builds while others wait; outputs are written under temporary names and moved into place
    with open(BUILD_DIR / "lock", "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        try:
            if not force and fresh():
                return module_path(), opt_path()
            tmp_mod = module_path().with_name(module_path().name + f".tmp{os.getpid()}")
            tmp_opt = opt_path().with_name(opt_path().name + f".tmp{os.getpid()}")
            cmds = [
                common + ["-shared", "-fvisibility=hidden", f"-I{pybind11.get_include()}",
                          f"-I{sysconfig.get_paths()['include']}", *lib, str(SRC_DIR / "bindings.cpp"), "-o", str(tmp_mod)],
                common + [*lib, str(SRC_DIR / "opt_main.cpp"), "-o", str(tmp_opt)],
            ]
            for cmd in cmds:
                res = subprocess.run(cmd, capture_output=True, text=True)
                if res.returncode != 0:
                    for t in (tmp_mod, tmp_opt):
                        if t.exists():
                            t.unlink()
                    raise RuntimeError(f"building the native compiler failed:\n{' '.join(cmd)}\n{res.stdout}\n{res.stderr}")
            os.replace(tmp_mod, module_path())
            os.replace(tmp_opt, opt_path())
            stamp_file.write_text(stamp)
        finally:
            fcntl.flock(lock, fcntl.LOCK_UN)
    return module_path(), opt_path()


def _source_digest() -> str:
    h = hashlib.sha256()
    for d in sorted(SRC_DIR.glob("*.cpp")) + sorted(SRC_DIR.glob("*.h")) + [ROOT / "csrc" / "runtime" / "json.h"]:
        h.update(d.read_bytes())
    return h.hexdigest()[:16]


def build_sanitized(out_dir=None) -> Path:
    """The command-line driver built with AddressSanitizer and UndefinedBehaviorSanitizer (aborting on the first
    finding), for running the pass pipeline over test IR on the host.  The reference has no sanitizer configuration;
    device-side sanitizers are not available for this code base, so the host-side C++ is checked this way."""
    out_dir = Path(out_dir) if out_dir is not None else BUILD_DIR / "sanitized"      # kept between runs: the build takes a while
    out_dir.mkdir(parents=True, exist_ok=True)
    out = out_dir / "nkipy-b200-opt-san"
    stamp, stamp_file = _source_digest(), out_dir / "stamp"
    if out.exists() and stamp_file.exists() and stamp_file.read_text() == stamp:
        return out
    cmd = ["g++", "-O1", "-g", "-std=c++17", "-Wall", "-fsanitize=address,undefined", "-fno-sanitize-recover=all",
           "-fno-omit-frame-pointer", str(SRC_DIR / "ir.cpp"), str(SRC_DIR / "passes.cpp"), str(SRC_DIR / "opt_main.cpp"),
           "-o", str(out)]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"building the sanitized driver failed:\n{' '.join(cmd)}\n{res.stdout}\n{res.stderr}")
    stamp_file.write_text(stamp)
    return out


def opt_main(argv=None) -> int:
    """Console entry `nkipy-b200-opt`: builds the native driver if needed and runs it with the given arguments
    (same role as the reference's `nkigen-opt`, nkigen/tools/nkigen-opt/nkigen-opt.cpp)."""
    _, exe = build()
    return subprocess.call([str(exe), *(sys.argv[1:] if argv is None else argv)])


if __name__ == "__main__":
    print(build(force="--force" in sys.argv))
