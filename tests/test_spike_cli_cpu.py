"""Argument handling of the spike-run CLI and compile-driver error surfacing (no GPU)."""
import subprocess

import numpy as np
import pytest

from nkipy_b200.core import compile as C
from nkipy_b200.spike import cli


def test_cli_parsing_and_env_validation(tmp_path, monkeypatch):
    np.save(tmp_path / "x_0.npy", np.ones(3))
    ins = cli.parse_inputs([f"x={tmp_path}/x_{{rank}}.npy"], 0)
    assert ins["x"].tolist() == [1, 1, 1]
    with pytest.raises(SystemExit):
        cli.parse_inputs(["nonsense"], 0)
    args = cli.build_parser().parse_args(["k.cubin", "--num-cores", "4", "--collective"])
    monkeypatch.setenv("CUDA_VISIBLE_DEVICES", "0,1")
    with pytest.raises(SystemExit):
        cli.validate_env(args)
    monkeypatch.setenv("CUDA_VISIBLE_DEVICES", "0,1,2,3")
    cli.validate_env(args)
    bad = cli.build_parser().parse_args(["k.cubin", "--cc-enabled", "--rank-id", "3", "--world-size", "2"])
    with pytest.raises(SystemExit):
        cli.validate_env(bad)


def test_compile_error_carries_command_and_output(monkeypatch, tmp_path):
    k = C.trace(lambda a: a * 2)
    k.specialize(np.zeros(4, np.float32))

    def fake_run(cmd, **kw):
        return subprocess.CompletedProcess(cmd, 1, stdout="some stdout", stderr="error: boom")

    cwd_before = __import__("os").getcwd()
    monkeypatch.setattr(C.subprocess, "run", fake_run)
    with pytest.raises(C.CompilationError) as ei:
        C.compile_to_neff(k, str(tmp_path))
    assert "boom" in str(ei.value) and "nvcc" in " ".join(ei.value.command) and ei.value.stdout == "some stdout"
    assert __import__("os").getcwd() == cwd_before
    with pytest.raises(RuntimeError):
        C.get_ir(C.trace(lambda a: a))


def test_compile_artifacts_and_lowering(tmp_path):
    def k(a, b):
        return np.exp(a) @ b

    path = C.compile_to_neff(C.trace(k).specialize(np.zeros((8, 16), np.float32), np.zeros((16, 4), np.float32)),
                             str(tmp_path), "k.neff", save_artifacts=True)
    assert path.endswith("k.cubin")
    names = sorted(p.name for p in tmp_path.iterdir())
    assert names == ["k.cu", "k.cubin", "k.ir.txt", "k.json"]
    src = C.lower_to_nki(k, np.zeros((8, 16), np.float32), np.zeros((16, 4), np.float32))
    assert "gemm_simt" in src and 'extern "C" __global__' in src
    assert C.get_platform_target() is C.CompilationTarget.SM100A
    C._set_build_dir(str(tmp_path / "b"))
    assert C._get_build_dir() == str(tmp_path / "b")
