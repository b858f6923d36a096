"""The packaging metadata names console scripts that exist and run."""
import importlib
import subprocess
import sys
import tomllib
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]


def _scripts():
    with open(ROOT / "pyproject.toml", "rb") as f:
        return tomllib.load(f)["project"]["scripts"]


def test_console_scripts_resolve():
    scripts = _scripts()
    assert {"spike-run", "nkipy-b200-opt"} <= set(scripts)
    for target in scripts.values():
        mod, fn = target.split(":")
        assert callable(getattr(importlib.import_module(mod), fn)), target


def test_opt_entry_runs_the_native_driver(tmp_path):
    from nkipy_b200.compiler.native import opt_main

    assert opt_main(["--list-passes"]) == 0
    out = subprocess.run([sys.executable, "-c", "from nkipy_b200.compiler.native import opt_main; import sys; "
                          "sys.exit(opt_main(['--list-passes']))"], capture_output=True, text=True, cwd=ROOT)
    assert out.returncode == 0 and "knob-driven-tiling" in out.stdout


def test_spike_run_help():
    out = subprocess.run([sys.executable, "-m", "nkipy_b200.spike.cli", "--help"], capture_output=True, text=True,
                         cwd=ROOT)
    assert out.returncode == 0 and "usage" in out.stdout.lower()


def test_concurrent_runtime_builds_compile_once_and_never_expose_a_partial_module(tmp_path):
    """Several rank processes that find the runtime module missing at the same time: one compiles under the build lock,
    the others wait and find it done; the module appears under its final name only when it is complete."""
    import os
    import textwrap

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    code = textwrap.dedent(f"""
        import subprocess, sys
        sys.path.insert(0, {root!r})
        from pathlib import Path
        from nkipy_b200.runtime import native
        native.OUT_DIR = Path({str(tmp_path)!r})
        native.BUILD_DIR = Path({str(tmp_path)!r}) / "build"
        calls = []
        real = subprocess.run
        def counting(cmd, *a, **kw):
            calls.append(cmd[0])
            return real(cmd, *a, **kw)
        native.subprocess.run = counting
        out = native.build()
        print(len(calls), out.exists(), out.stat().st_size > 100000)
    """)
    procs = [subprocess.Popen([sys.executable, "-c", code], stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True)
             for _ in range(4)]
    outs = [p.communicate(timeout=600) for p in procs]
    assert all(p.returncode == 0 for p in procs), outs
    counts = sorted(int(o[0].split()[0]) for o in outs)
    assert counts == [0, 0, 0, 1], counts
    assert all(o[0].split()[1:] == ["True", "True"] for o in outs)
    assert not [f for f in os.listdir(tmp_path) if ".tmp" in f]
