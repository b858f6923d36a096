"""kernel_agent: catalogue, three-stage executor, offline generator, sweep + rerun."""
import json
import os

import numpy as np
import pytest

from nkipy_b200.tools.kernel_agent import ops as ka_ops
from nkipy_b200.tools.kernel_agent.__main__ import main
from nkipy_b200.tools.kernel_agent.executor import run_kernel
from nkipy_b200.tools.kernel_agent.generator import BedrockClient, TemplateClient, load_kernel
from nkipy_b200.tools.kernel_agent.sweep import rerun_failed, run_sweep


def test_catalogue_ops_pass_without_gpu():
    table = ka_ops.discover(use_gpu=False)
    bad = {k: v for k, v in table.items() if v["status"] != "pass"}
    assert not bad, bad
    assert len(table) >= 60


def test_executor_reports_the_failing_stage():
    r = run_kernel(lambda a: a @ np.ones((3, 3), np.float32), [np.ones((4, 5), np.float32)], use_gpu=False)
    assert not r.passed and r.error_stage == "numpy"
    r = run_kernel(lambda a: np.exp(a) / np.sum(np.exp(a), -1, keepdims=True), [np.ones((4, 5), np.float32)],
                   use_gpu=False)
    assert r.passed and r.compile_ok and r.hardware_ok is None


def test_generator_and_cli(tmp_path, capsys):
    src = TemplateClient().generate(["exp", "multiply", "max", "where"], "")
    kernel, make_inputs = load_kernel(src)
    assert run_kernel(kernel, make_inputs(), use_gpu=False).passed
    with pytest.raises(RuntimeError):
        BedrockClient().generate(["exp"], "")
    f = tmp_path / "k.py"
    assert main(["generate", "tanh", "add", "-o", str(f)]) == 0
    assert main(["test", str(f), "--no-gpu"]) == 0
    assert main(["list-ops"]) == 0
    assert "binary:" in capsys.readouterr().out


def test_sweep_and_rerun(tmp_path):
    s = run_sweep(4, 3, str(tmp_path), seed=1, use_gpu=False)
    assert s["passed"] == 4 and os.path.exists(tmp_path / "sweep_results.json")
    # mark one as failed and let rerun fix the record
    data = json.load(open(tmp_path / "sweep_results.json"))
    data["results"][0]["passed"] = False
    json.dump(data, open(tmp_path / "sweep_results.json", "w"))
    assert rerun_failed(str(tmp_path), use_gpu=False)["passed"] == 4


@pytest.mark.gpu
def test_sweep_on_device(tmp_path):
    s = run_sweep(3, 4, str(tmp_path), seed=2)
    assert s["passed"] == 3, s
    assert all(r["hardware_ok"] for r in s["results"])
