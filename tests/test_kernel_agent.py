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


def test_sweep_log_is_jsonl_with_full_records(tmp_path):
    from nkipy_b200.tools.kernel_agent import SweepRecord, load_records, run_rerun

    s = run_sweep(3, 3, str(tmp_path), seed=3, use_gpu=False)
    recs = load_records(s["log"])
    assert len(recs) == 3 and all(isinstance(r, SweepRecord) for r in recs)
    r = recs[0]
    assert r.passed and r.numpy_success and r.compile_success and r.hardware_success is None
    assert "def kernel" in r.generated_code and r.input_specs["arg0"]["shape"]
    assert r.duration_seconds >= 0 and r.timestamp.endswith("Z")
    # a torn last line (killed writer) is skipped, not fatal
    with open(s["log"], "a") as f:
        f.write('{"iteration": 9, "times')
    assert len(load_records(s["log"])) == 3
    # replay from the saved source
    again = run_rerun(s["log"], use_gpu=False, out_dir=str(tmp_path / "again"))
    assert again["passed"] == 3 and again["results"][0]["rerun_source"] == os.path.basename(s["log"])
    with pytest.raises(ValueError):
        run_rerun(str(tmp_path / "sweep_results.json"), use_gpu=False)
    with pytest.raises(FileNotFoundError):
        run_rerun(str(tmp_path / "missing.jsonl"), use_gpu=False)


class _SlowClient:
    """Generator stand-in whose second kernel never finishes on its own."""
    model_id = "slow"

    def __init__(self):
        self.inner, self.calls = TemplateClient(0), 0

    def generate(self, ops, prompt):
        self.calls += 1
        if self.calls == 2:
            import time
            time.sleep(30)
        return self.inner.generate(ops, prompt)


def test_sweep_abandons_an_iteration_that_exceeds_its_timeout(tmp_path):
    s = run_sweep(3, 2, str(tmp_path), seed=4, use_gpu=False, client=_SlowClient(), timeout=1)
    assert [r["passed"] for r in s["results"]] == [True, False, True]
    assert s["results"][1]["failure_stage"] == "timeout" and s["failed_by_stage"] == {"timeout": 1}


class _InterruptingClient:
    """Sends this process SIGTERM while the second kernel is generated."""
    model_id = "interrupt"

    def __init__(self):
        self.inner, self.calls = TemplateClient(0), 0

    def generate(self, ops, prompt):
        import signal
        self.calls += 1
        if self.calls == 2:
            os.kill(os.getpid(), signal.SIGTERM)
        return self.inner.generate(ops, prompt)


def test_sweep_stops_gracefully_on_sigterm_and_restores_handlers(tmp_path):
    import signal
    before = signal.getsignal(signal.SIGTERM)
    s = run_sweep(None, 2, str(tmp_path), seed=5, use_gpu=False, client=_InterruptingClient())
    # the iteration in flight is finished and logged, then the sweep returns
    assert s["interrupted"] and s["num_kernels"] == 2 and s["passed"] == 2
    assert signal.getsignal(signal.SIGTERM) is before
    from nkipy_b200.tools.kernel_agent import load_records
    assert len(load_records(s["log"])) == 2


def test_generation_failure_is_a_record_not_a_crash(tmp_path):
    s = run_sweep(2, 2, str(tmp_path), seed=6, use_gpu=False, client=BedrockClient())
    assert s["passed"] == 0 and s["failed_by_stage"] == {"generate": 2}
