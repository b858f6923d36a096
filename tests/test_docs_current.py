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
