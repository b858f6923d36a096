"""The type stub of the runtime bindings stays in step with the C++ source that defines them."""
import ast
import re
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
BINDINGS = ROOT / "csrc" / "runtime" / "bindings.cpp"
STUB = ROOT / "nkipy_b200" / "spike" / "_spike.pyi"


def _bound_names():
    """{class: {member}} from the pybind11 source (`py::class_<...>(m, "Name")` followed by `.def*("member"`)."""
    src = BINDINGS.read_text()
    out = {}
    parts = re.split(r'py::class_<[^;]*?>\(m,\s*"(\w+)"\)', src)
    for name, body in zip(parts[1::2], parts[2::2]):
        body = body.split("py::class_<")[0]
        members = set(re.findall(r'\.def(?:_static|_property_readonly|_readonly|_readwrite)?\(\s*"(\w+)"', body))
        out[name] = members
    return out


def _stub_names():
    tree = ast.parse(STUB.read_text())
    out = {}
    for node in tree.body:
        if isinstance(node, ast.ClassDef):
            out[node.name] = {n.name for n in node.body if isinstance(n, ast.FunctionDef)}
    return out


def test_stub_lists_every_bound_class_and_member():
    bound, stub = _bound_names(), _stub_names()
    assert set(bound) <= set(stub), set(bound) - set(stub)
    for cls, members in bound.items():
        have = stub[cls] | ({"__init__"} if "__init__" in stub[cls] else set())
        missing = members - have
        assert not missing, (cls, missing)


def test_stub_declares_nothing_the_bindings_lack():
    bound, stub = _bound_names(), _stub_names()
    for cls, members in stub.items():
        if cls not in bound:
            assert cls in ("SpikeRuntimeError", "SpikeError", "CudaError"), cls
            continue
        extra = {m for m in members if m != "__init__"} - bound[cls]
        assert not extra, (cls, extra)


def test_stub_matches_the_built_module_when_present():
    try:
        from nkipy_b200.spike import _spike
    except Exception:
        return
    for cls, members in _stub_names().items():
        obj = getattr(_spike, cls)
        for m in members:
            if m != "__init__":
                assert hasattr(obj, m), (cls, m)
