// pybind11 module `_spike`: Python surface of the device runtime, shaped like the
// reference's nanobind module (spike/src/python_bindings.cpp:23-219): exception types,
// SystemTraceSession context manager, TensorMetadata / ModelTensorInfo, NrtTensor /
// NrtModel handles and the Spike facade; execute releases the GIL; tensor writes take any
// buffer-protocol object without copying, reads fill a caller-provided buffer or return bytes.
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include "spike.h"
#include "symmetric.h"

namespace py = pybind11;
using namespace spike;

PYBIND11_MODULE(_spike, m) {
  m.doc() = "CUDA-driver device runtime (tensors, cubin modules, execution, tracing)";

  static py::exception<SpikeRuntimeError> ex_runtime(m, "SpikeRuntimeError", PyExc_RuntimeError);
  static py::exception<SpikeError> ex_spike(m, "SpikeError", ex_runtime.ptr());
  static py::exception<CudaError> ex_cuda(m, "CudaError", ex_runtime.ptr());
  m.attr("NrtError") = m.attr("CudaError");
  py::register_exception_translator([](std::exception_ptr p) {
    try {
      if (p) std::rethrow_exception(p);
    } catch (const CudaError& e) {
      // the driver's status code travels with the exception (`e.code`), as the vendor code does in the reference
      py::object exc = py::reinterpret_borrow<py::object>(ex_cuda.ptr())(e.what());
      exc.attr("code") = e.code();
      PyErr_SetObject(ex_cuda.ptr(), exc.ptr());
    } catch (const SpikeError& e) {
      PyErr_SetString(ex_spike.ptr(), e.what());
    } catch (const SpikeRuntimeError& e) {
      PyErr_SetString(ex_runtime.ptr(), e.what());
    }
  });

  py::class_<TraceSession>(m, "SystemTraceSession")
      .def(py::init<int, size_t>(), py::arg("core_id") = -1, py::arg("capacity") = 65536)
      .def("stop", &TraceSession::stop)
      .def("fetch_events_json", &TraceSession::fetch_events_json)
      .def("drain_events", &TraceSession::drain_events)
      .def_property_readonly("active", &TraceSession::active)
      .def("__enter__", [](TraceSession& s) -> TraceSession& { return s; }, py::return_value_policy::reference)
      .def("__exit__", [](TraceSession& s, py::object, py::object, py::object) { s.stop(); });

  py::class_<TensorMetadata>(m, "TensorMetadata")
      .def_readonly("size", &TensorMetadata::size)
      .def_readonly("dtype", &TensorMetadata::dtype)
      .def_readonly("shape", &TensorMetadata::shape)
      .def("__repr__", [](const TensorMetadata& t) {
        std::string s = "TensorMetadata(size=" + std::to_string(t.size) + ", dtype='" + t.dtype + "', shape=[";
        for (size_t i = 0; i < t.shape.size(); ++i) s += (i ? ", " : "") + std::to_string(t.shape[i]);
        return s + "])";
      });

  py::class_<ModelTensorInfo>(m, "ModelTensorInfo")
      .def_readonly("inputs", &ModelTensorInfo::inputs)
      .def_readonly("outputs", &ModelTensorInfo::outputs)
      .def_readonly("input_order", &ModelTensorInfo::input_order)
      .def_readonly("output_order", &ModelTensorInfo::output_order)
      .def_readonly("aliases", &ModelTensorInfo::aliases);

  py::class_<DeviceBuffer, std::shared_ptr<DeviceBuffer>>(m, "NrtTensor")
      .def_property_readonly("core_id", &DeviceBuffer::core_id)
      .def_property_readonly("size", &DeviceBuffer::size)
      .def_property_readonly("name", &DeviceBuffer::name)
      .def_property_readonly("va", &DeviceBuffer::va)
      .def_property_readonly("is_freed", &DeviceBuffer::is_freed);

  py::class_<LoadedModule, std::shared_ptr<LoadedModule>>(m, "NrtModel")
      .def_property_readonly("neff_path", &LoadedModule::path)
      .def_property_readonly("name", &LoadedModule::name)
      .def_property_readonly("core_id", &LoadedModule::core_id)
      .def_property_readonly("rank_id", &LoadedModule::rank_id)
      .def_property_readonly("world_size", &LoadedModule::world_size)
      .def_property_readonly("is_collective", &LoadedModule::is_collective)
      .def_property_readonly("num_launches", &LoadedModule::num_launches)
      .def_property_readonly("has_collectives", &LoadedModule::has_collectives)
      .def_property_readonly("collective_world", &LoadedModule::collective_world)
      .def_property_readonly("workspace_bytes", &LoadedModule::workspace_bytes)
      .def("set_collective_workspace", &LoadedModule::set_collective_workspace, py::arg("peer_ws"))
      .def_property_readonly("unloaded", &LoadedModule::unloaded);

  py::class_<SymmetricBuffer>(m, "SymmetricBuffer")
      .def(py::init<int, size_t>(), py::arg("device_ordinal"), py::arg("bytes"))
      .def_static("supported", &SymmetricBuffer::supported)
      .def_static("multicast_supported", &SymmetricBuffer::multicast_supported)
      .def_property_readonly("size", &SymmetricBuffer::size)
      .def_property_readonly("device_ordinal", &SymmetricBuffer::device_ordinal)
      .def_property_readonly("local_ptr", &SymmetricBuffer::local_ptr)
      .def_property_readonly("multicast_ptr", &SymmetricBuffer::multicast_ptr)
      .def_property_readonly("has_multicast", &SymmetricBuffer::has_multicast)
      .def_property_readonly("closed", &SymmetricBuffer::closed)
      .def("export_fd", &SymmetricBuffer::export_fd)
      .def("import_peer", &SymmetricBuffer::import_peer, py::arg("rank"), py::arg("fd"))
      .def("peer_ptr", &SymmetricBuffer::peer_ptr, py::arg("rank"))
      .def("multicast_create", &SymmetricBuffer::multicast_create, py::arg("num_devices"))
      .def("multicast_import", &SymmetricBuffer::multicast_import, py::arg("fd"))
      .def("multicast_add_device", &SymmetricBuffer::multicast_add_device)
      .def("multicast_bind", &SymmetricBuffer::multicast_bind)
      .def("zero", &SymmetricBuffer::zero)
      .def("close", &SymmetricBuffer::close);

  py::class_<Spike>(m, "Spike")
      .def(py::init<int, int>(), py::arg("verbose_level") = 0, py::arg("device_ordinal") = -1)
      .def_static("get_visible_neuron_core_count", &Spike::get_visible_neuron_core_count)
      .def_property_readonly("device_ordinal", &Spike::device_ordinal)
      .def_property_readonly("device_name", &Spike::device_name)
      .def_property_readonly("sm_count", &Spike::sm_count)
      .def_property_readonly("total_memory", &Spike::total_memory)
      .def_property_readonly("is_closed", &Spike::is_closed)
      .def("load_model", &Spike::load_model, py::arg("neff_path"), py::arg("core_id") = 0,
           py::arg("cc_enabled") = false, py::arg("rank_id") = 0, py::arg("world_size") = 1)
      .def("unload_model", &Spike::unload_model)
      .def("allocate_tensor", &Spike::allocate_tensor, py::arg("size"), py::arg("core_id") = 0,
           py::arg("name") = std::string())
      .def("slice_from_tensor", &Spike::slice_from_tensor, py::arg("source"), py::arg("offset"), py::arg("size"),
           py::arg("name") = std::string())
      .def("free_tensor", &Spike::free_tensor)
      .def("tensor_write",
           [](Spike& s, const std::shared_ptr<DeviceBuffer>& t, py::buffer data, size_t offset) {
             py::buffer_info info = data.request();
             size_t nbytes = static_cast<size_t>(info.size) * static_cast<size_t>(info.itemsize);
             if (!PyBuffer_IsContiguous(info.view(), 'C')) throw SpikeError("tensor_write needs a C-contiguous buffer");
             const void* ptr = info.ptr;
             py::gil_scoped_release release;
             s.tensor_write(t, ptr, nbytes, offset);
           },
           py::arg("tensor"), py::arg("data"), py::arg("offset") = 0)
      .def("tensor_read",
           [](Spike& s, const std::shared_ptr<DeviceBuffer>& t, size_t offset, size_t size) {
             std::string out(size, '\0');
             {
               py::gil_scoped_release release;
               s.tensor_read(t, out.data(), size, offset);
             }
             return py::bytes(out);
           },
           py::arg("tensor"), py::arg("offset") = 0, py::arg("size") = 0)
      .def("tensor_read_to_buffer",
           [](Spike& s, const std::shared_ptr<DeviceBuffer>& t, py::buffer dest, size_t offset) {
             py::buffer_info info = dest.request(true);
             size_t nbytes = static_cast<size_t>(info.size) * static_cast<size_t>(info.itemsize);
             if (!PyBuffer_IsContiguous(info.view(), 'C')) throw SpikeError("tensor_read needs a C-contiguous buffer");
             void* ptr = info.ptr;
             py::gil_scoped_release release;
             s.tensor_read(t, ptr, nbytes, offset);
           },
           py::arg("tensor"), py::arg("dest"), py::arg("offset") = 0)
      .def("execute",
           [](Spike& s, const std::shared_ptr<LoadedModule>& model,
              const std::map<std::string, std::shared_ptr<DeviceBuffer>>& inputs,
              const std::map<std::string, std::shared_ptr<DeviceBuffer>>& outputs, const std::string& ntff_name,
              bool save_trace) {
             std::vector<std::pair<std::string, std::shared_ptr<DeviceBuffer>>> in(inputs.begin(), inputs.end());
             std::vector<std::pair<std::string, std::shared_ptr<DeviceBuffer>>> out(outputs.begin(), outputs.end());
             py::gil_scoped_release release;
             s.execute(model, in, out, ntff_name, save_trace);
           },
           py::arg("model"), py::arg("inputs"), py::arg("outputs"), py::arg("ntff_name") = std::string(),
           py::arg("save_trace") = false)
      .def("get_tensor_info", &Spike::get_tensor_info)
      .def("read_status", &Spike::read_status, py::arg("reset") = true)
      .def("close", [](Spike& s) { s.close(); return 0; });   // 0 = success, like the other status-returning calls
}
