"""The generated operation reference under docs/api is what the generator produces from the current registry."""
import importlib.util
import os

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _generator():
    spec = importlib.util.spec_from_file_location("generate_api_docs", os.path.join(ROOT, "docs", "generate_api_docs.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_committed_api_reference_is_current(tmp_path):
    gen = _generator()
    for fname, writer in (("ops.md", gen.write_ops), ("numpy_compat.md", gen.write_numpy)):
        out = tmp_path / fname
        assert writer(str(out)) > 0
        committed = open(os.path.join(ROOT, "docs", "api", fname)).read()
        assert out.read_text() == committed, f"docs/api/{fname} is stale: run python docs/generate_api_docs.py"


def test_python_blocks_of_the_custom_kernel_tutorial_run_on_the_cpu():
    import re

    text = open(os.path.join(ROOT, "docs", "tutorials", "custom_kernel.md")).read()
    blocks = re.findall(r"```python\n(.*?)```", text, re.S)
    assert len(blocks) >= 4
    scope = {}
    for block in blocks:                      # later blocks use names the earlier ones define
        exec(compile(block, "custom_kernel.md", "exec"), scope)


def test_every_tutorial_is_linked_from_the_index():
    folder = os.path.join(ROOT, "docs", "tutorials")
    index = open(os.path.join(folder, "index.md")).read()
    for name in os.listdir(folder):
        if name.endswith(".md") and name != "index.md":
            assert f"({name})" in index, f"{name} is not linked from docs/tutorials/index.md"
