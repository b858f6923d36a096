// pybind11 module `_b200c`: in-process access to the native pass pipeline (the reference
// exposes its passes through MLIR Python bindings, nkigen/mlir/lib/Bindings/NkipyModule.cpp).
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include "passes.h"

namespace py = pybind11;
using namespace b200c;

static PassOptions make_options(long long smem_capacity, long long tmem_columns, int sm_count, bool fast_math) {
  PassOptions o;
  o.smem_capacity = smem_capacity;
  o.tmem_columns = tmem_columns;
  o.sm_count = sm_count;
  o.fast_math = fast_math;
  return o;
}

PYBIND11_MODULE(_b200c, m) {
  m.doc() = "native tensor-IR pass pipeline";
  static py::exception<CompileError> ex(m, "CompileError", PyExc_RuntimeError);
  m.def("apply_passes",
        [](const std::string& ir, const std::vector<std::string>& passes, long long smem, long long tmem, int sms,
           bool fast) { return apply_passes(ir, passes, make_options(smem, tmem, sms, fast)); },
        py::arg("ir_text"), py::arg("passes"), py::arg("smem_capacity") = 232448, py::arg("tmem_columns") = 512,
        py::arg("sm_count") = 148, py::arg("fast_math") = false);
  m.def("run_pipeline",
        [](const std::string& ir, const std::string& stop_after, const std::string& dump_dir, long long smem,
           long long tmem, int sms, bool fast, int dump_start) {
          return run_pipeline(ir, stop_after, dump_dir, make_options(smem, tmem, sms, fast), dump_start);
        },
        py::arg("ir_text"), py::arg("stop_after") = "", py::arg("dump_dir") = "", py::arg("smem_capacity") = 232448,
        py::arg("tmem_columns") = 512, py::arg("sm_count") = 148, py::arg("fast_math") = false,
        py::arg("dump_start") = 1);
  m.def("list_passes", [] {
    std::vector<std::tuple<std::string, std::string, std::string>> out;
    for (const PassInfo& p : default_pipeline()) out.emplace_back(p.name, p.group, p.description);
    return out;
  });
  m.def("verify", [](const std::string& ir) {
    auto g = Graph::parse(ir);
    g->verify();
    return g->print();
  });
}
