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
