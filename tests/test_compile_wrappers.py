"""`compile_to_neff` / `lower_to_nki` / `Compiler`: what they write, how the cache directory is laid out and
how a failing nvcc run is reported (counterpart of the reference's tests/unit/test_compile_wrappers.py)."""
import json
import os
import subprocess
from pathlib import Path
from types import SimpleNamespace

import numpy as np
import pytest

from nkipy_b200.core import compile as C
from nkipy_b200.core.compile import (CompilationConfig, CompilationError, CompilationTarget, Compiler, compile_to_neff,
                                     lower_to_nki, trace)


def softmax_kernel(x):
    e = np.exp(x - np.max(x, axis=-1, keepdims=True))
    return e / np.sum(e, axis=-1, keepdims=True)


@pytest.fixture
def kernel():
    k = trace(softmax_kernel)
    k.specialize(np.ones((8, 64), np.float32))
    return k


def test_compile_to_neff_writes_cubin_and_plan(kernel, tmp_path):
    path = compile_to_neff(kernel, str(tmp_path), "softmax.cubin")
    assert path == str(tmp_path / "softmax.cubin") and os.path.getsize(path) > 0
    plan = json.load(open(tmp_path / "softmax.json"))
    assert plan["launches"] and plan["inputs"] and plan["outputs"]
    assert not (tmp_path / "softmax.cu").exists()                    # no artifacts unless asked


def test_a_neff_name_is_accepted_and_mapped_to_a_cubin(kernel, tmp_path):
    path = compile_to_neff(kernel, str(tmp_path), "file.neff")
    assert path.endswith("file.cubin") and os.path.exists(path)


def test_compile_to_neff_with_artifacts(kernel, tmp_path):
    compile_to_neff(kernel, str(tmp_path), "k.cubin", save_artifacts=True)
    src = (tmp_path / "k.cu").read_text()
    assert "__global__" in src and (tmp_path / "k.ir.txt").read_text().startswith("graph")


@pytest.mark.parametrize("target", [CompilationTarget.DEFAULT, CompilationTarget.SM100A, CompilationTarget.TRN2])
def test_every_target_builds_for_sm100a(kernel, tmp_path, target, monkeypatch):
    seen = {}
    real = subprocess.run

    def spy(cmd, **kw):
        seen["cmd"] = cmd
        return real(cmd, **kw)

    monkeypatch.setattr(C.subprocess, "run", spy)
    compile_to_neff(kernel, str(tmp_path / target.name), "k.cubin", target=target)
    assert "arch=compute_100a,code=sm_100a" in seen["cmd"] and "-lineinfo" in seen["cmd"]


def test_additional_compiler_args_reach_nvcc(kernel, tmp_path, monkeypatch):
    seen = {}
    real = subprocess.run

    def spy(cmd, **kw):
        seen["cmd"] = cmd
        return real(cmd, **kw)

    monkeypatch.setattr(C.subprocess, "run", spy)
    compile_to_neff(kernel, str(tmp_path), "k.cubin", additional_compiler_args="-O1 --use_fast_math")
    assert "-O1" in seen["cmd"] and "--use_fast_math" in seen["cmd"] and "-O3" not in seen["cmd"]


def test_lower_to_nki_returns_source(kernel):
    src = lower_to_nki(kernel)
    assert "__global__" in src and "expf" in src
    # a plain function plus arguments is traced on the fly
    assert "__global__" in lower_to_nki(softmax_kernel, np.ones((4, 32), np.float32))


def test_unspecialized_kernel_is_rejected(tmp_path):
    with pytest.raises(RuntimeError, match="specialize"):
        compile_to_neff(trace(softmax_kernel), str(tmp_path))


def test_output_directory_that_cannot_be_created(kernel, tmp_path):
    blocker = tmp_path / "file"
    blocker.write_text("not a directory")
    with pytest.raises(OSError):
        compile_to_neff(kernel, str(blocker / "sub"), "k.cubin")


# ----------------------------------------------------------------------------- error surfacing
def _fake_run(returncode, stdout="", stderr="", make_output=False):
    def run(cmd, **kw):
        if make_output:
            Path(cmd[cmd.index("-o") + 1]).write_bytes(b"cubin")
        return SimpleNamespace(returncode=returncode, stdout=stdout, stderr=stderr)
    return run


def test_nonzero_exit_surfaces_command_stderr_and_stdout(kernel, tmp_path, monkeypatch):
    monkeypatch.setattr(C.subprocess, "run", _fake_run(1, "compiling...\n", "error: identifier undefined\n"))
    with pytest.raises(CompilationError) as e:
        Compiler(CompilationConfig()).compile_graph(C.get_ir(kernel), str(tmp_path), "k.cubin")
    msg = str(e.value)
    assert "exit code 1" in msg and "identifier undefined" in msg and "compiling..." in msg and "nvcc" in msg
    assert e.value.stderr.startswith("error:") and e.value.command[0].endswith("nvcc")
    assert not (tmp_path / "k.json").exists()                        # no launch plan for a kernel that did not build


def test_zero_exit_without_output_is_an_error(kernel, tmp_path, monkeypatch):
    monkeypatch.setattr(C.subprocess, "run", _fake_run(0, "", "warning: nothing emitted\n"))
    with pytest.raises(CompilationError, match="expected but not generated") as e:
        Compiler().compile_graph(C.get_ir(kernel), str(tmp_path), "k.cubin")
    assert "nothing emitted" in str(e.value)


def test_success_returns_the_paths(kernel, tmp_path, monkeypatch):
    monkeypatch.setattr(C.subprocess, "run", _fake_run(0, make_output=True))
    res = Compiler().compile_graph(C.get_ir(kernel), str(tmp_path), "k.cubin")
    assert res.neff_path == str(tmp_path / "k.cubin") == res.cubin_path and res.plan_path == str(tmp_path / "k.json")
    assert res.work_dir == str(tmp_path) and res.source_path is None


def test_working_directory_survives_a_failure(kernel, tmp_path, monkeypatch):
    monkeypatch.setattr(C.subprocess, "run", _fake_run(1))
    before = os.getcwd()
    with pytest.raises(CompilationError):
        Compiler().compile_graph(C.get_ir(kernel), str(tmp_path), "k.cubin")
    assert os.getcwd() == before


def test_missing_nvcc_is_reported(kernel, tmp_path, monkeypatch):
    monkeypatch.setattr(C.shutil, "which", lambda name: None)
    monkeypatch.setattr(C.os.path, "exists", lambda p: False if "nvcc" in str(p) else os.path.lexists(p))
    monkeypatch.delenv("NVCC", raising=False)
    with pytest.raises(CompilationError, match="nvcc not found"):
        Compiler()._command(tmp_path / "a.cu", tmp_path / "a.cubin")
