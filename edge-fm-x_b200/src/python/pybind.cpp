// Python module `edge_fm`: Tensor, Request, Response, EdgeFM, enums and the exception tree.
// Same names, constructors and exception mapping as the reference module
// (src/python/pybind.cpp:90-258) plus the Tensor helpers its tests use from the debug variant
// (data_ptr / to_dlpack / MemoryOwnership: src/python/pybind_debug.cpp:364-481).
#include <Python.h>
#include <dlpack/dlpack.h>
#include <edge-fm/core.h>
#include <edge-fm/edge-fm.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include <cstdint>

namespace py = pybind11;
using namespace edge_fm;

namespace {

Tensor tensor_from_address(uintptr_t data_ptr, const std::vector<int64_t>& shape, DType dtype, Device device,
                           int32_t device_id, bool copy_data) {
    void* p = reinterpret_cast<void*>(data_ptr);
    if (!copy_data) return Tensor::view(p, shape, dtype, device, device_id);
    return Tensor::clone_from(p, shape, dtype, device, device_id, device, device_id,
                              device == Device::GPU ? MemoryOwnership::OwnCudaMalloc : MemoryOwnership::OwnCpuMalloc, nullptr);
}

Tensor tensor_from_capsule(py::object capsule) {
    if (!PyCapsule_CheckExact(capsule.ptr())) throw std::runtime_error("Expected a PyCapsule object for DLPack tensor");
    const char* name = PyCapsule_GetName(capsule.ptr());
    if (name == nullptr || std::string(name) != "dltensor") throw std::runtime_error("Invalid DLPack capsule name. Expected 'dltensor'");
    auto* mt = static_cast<DLManagedTensor*>(PyCapsule_GetPointer(capsule.ptr(), "dltensor"));
    if (mt == nullptr) throw std::runtime_error("Failed to get DLManagedTensor from capsule");
    return Tensor::from_dlpack(mt);     // copies; the capsule stays owned by its producer
}

py::capsule tensor_to_capsule(const Tensor& t) {
    DLManagedTensor* mt = t.to_dlpack();
    return py::capsule(mt, "dltensor", [](PyObject* cap) {
        if (PyCapsule_IsValid(cap, "dltensor")) {        // never consumed: release it ourselves
            auto* m = static_cast<DLManagedTensor*>(PyCapsule_GetPointer(cap, "dltensor"));
            if (m != nullptr && m->deleter != nullptr) m->deleter(m);
        }
    });
}

// dict[str, Tensor] -> pointers into the Python-owned tensors (alive for the duration of the call), and back:
// the conversions of the reference's planner bindings (src/python/pybind_debug.cpp:108-130,1672-1679).
TensorRefMap tensor_ref_map_from_py_dict(const py::dict& dict) {
    TensorRefMap out;
    for (auto item : dict) {
        const std::string key = py::cast<std::string>(item.first);
        out[key] = &py::cast<const Tensor&>(item.second);
    }
    return out;
}

py::dict tensor_map_to_py_dict(TensorMap&& map) {
    py::dict out;
    for (auto& kv : map) out[py::str(kv.first)] = py::cast(new Tensor(std::move(kv.second)), py::return_value_policy::take_ownership);
    return out;
}

}  // namespace

PYBIND11_MODULE(edge_fm, m) {
    m.doc() = "EdgeFM single-request inference engine (B200 backend)";

    static py::exception<Error> err(m, "Error", PyExc_RuntimeError);
    py::register_exception<DeviceError>(m, "DeviceError", err.ptr());
    py::register_exception<ConfigurationError>(m, "ConfigurationError", err.ptr());
    py::register_exception<ModelNotLoadedError>(m, "ModelNotLoadedError", err.ptr());
    py::register_exception<InvalidRequestError>(m, "InvalidRequestError", err.ptr());
    py::register_exception<OutOfMemoryError>(m, "OutOfMemoryError", err.ptr());
    py::register_exception<InternalError>(m, "InternalError", err.ptr());
    // Callers of the reference catch builtin exception types: keep its mapping on top.
    py::register_exception_translator([](std::exception_ptr p) {
        try {
            if (p) std::rethrow_exception(p);
        } catch (const DeviceError& e) { PyErr_SetString(PyExc_RuntimeError, e.what());
        } catch (const ConfigurationError& e) { PyErr_SetString(PyExc_ValueError, e.what());
        } catch (const ModelNotLoadedError& e) { PyErr_SetString(PyExc_RuntimeError, e.what());
        } catch (const InvalidRequestError& e) { PyErr_SetString(PyExc_ValueError, e.what());
        } catch (const OutOfMemoryError& e) { PyErr_SetString(PyExc_MemoryError, e.what());
        } catch (const InternalError& e) { PyErr_SetString(PyExc_RuntimeError, e.what());
        }
    });

    py::enum_<Device>(m, "Device").value("CPU", Device::CPU).value("GPU", Device::GPU).export_values();
    py::enum_<DType>(m, "DType")
        .value("Float32", DType::Float32).value("Float16", DType::Float16).value("BFloat16", DType::BFloat16)
        .value("Int32", DType::Int32).value("Int64", DType::Int64).value("UInt8", DType::UInt8).value("Int8", DType::Int8)
        .export_values();
    // which of a model's two weight sets / passes a call refers to (reference: src/engine/engine.h:16, bound at
    // src/python/pybind_debug.cpp:349-351)
    py::enum_<ModelStage>(m, "ModelStage").value("Prefill", ModelStage::Prefill).value("Decode", ModelStage::Decode);
    py::enum_<MemoryOwnership>(m, "MemoryOwnership")
        .value("ViewExternal", MemoryOwnership::ViewExternal).value("OwnCpuMalloc", MemoryOwnership::OwnCpuMalloc)
        .value("OwnCudaMalloc", MemoryOwnership::OwnCudaMalloc).value("OwnCudaPool", MemoryOwnership::OwnCudaPool);

    py::class_<Tensor>(m, "Tensor")
        .def(py::init(&tensor_from_address), py::arg("data_ptr"), py::arg("shape"), py::arg("dtype"), py::arg("device"),
             py::arg("device_id") = 0, py::arg("copy_data") = false,
             "Wrap (copy_data=False) or copy (copy_data=True) a contiguous row-major buffer given by address")
        .def_static("from_dlpack", &tensor_from_capsule, py::arg("capsule"), "Copy a DLPack capsule into a new Tensor")
        .def("to_dlpack", &tensor_to_capsule, "Export as a DLPack capsule sharing this tensor's buffer")
        .def("empty", &Tensor::empty)
        .def("dtype", &Tensor::dtype)
        .def("shape", &Tensor::shape)
        .def("device", &Tensor::device)
        .def("data_ptr", [](const Tensor& t) { return reinterpret_cast<uintptr_t>(t.data_ptr()); })
        .def("dump", &Tensor::dump, py::arg("file_path"));

    py::class_<Request>(m, "Request")
        .def(py::init<int, const std::vector<int32_t>&>(), py::arg("request_id"), py::arg("token_ids"))
        // device / device_id: where the request's deep copies of embedding and position_ids are placed (multi-GPU callers
        // pass their own GPU; the defaults are the reference's: GPU 0)
        .def(py::init([](int id, const std::vector<int32_t>& ids, const Tensor& emb, int32_t eid, Device dev, int32_t dev_id) {
                 return new Request(id, ids, emb, eid, dev, dev_id);
             }),
             py::arg("request_id"), py::arg("token_ids"), py::arg("embedding"), py::arg("embed_token_id") = -1,
             py::arg("device") = Device::GPU, py::arg("device_id") = 0)
        .def(py::init([](int id, const std::vector<int32_t>& ids, const Tensor& emb, int32_t eid, const Tensor& pos, Device dev, int32_t dev_id) {
                 return new Request(id, ids, emb, eid, pos, dev, dev_id);
             }),
             py::arg("request_id"), py::arg("token_ids"), py::arg("embedding"), py::arg("embed_token_id"), py::arg("position_ids"),
             py::arg("device") = Device::GPU, py::arg("device_id") = 0)
        .def(py::init([](int id, const std::vector<int32_t>& ids, const Tensor& emb, int32_t eid, const Tensor& pos,
                         const std::vector<int32_t>& last, Device dev, int32_t dev_id) {
                 return new Request(id, ids, emb, eid, pos, last, dev, dev_id);
             }),
             py::arg("request_id"), py::arg("token_ids"), py::arg("embedding"), py::arg("embed_token_id"), py::arg("position_ids"),
             py::arg("mrope_last_pos"), py::arg("device") = Device::GPU, py::arg("device_id") = 0)
        .def("request_id", &Request::request_id)
        .def("token_ids", &Request::token_ids, py::return_value_policy::reference_internal)
        .def("embedding", &Request::embedding, py::return_value_policy::reference_internal)
        .def("embed_token_id", &Request::embed_token_id)
        .def("has_embedding", &Request::has_embedding)
        .def("position_ids", &Request::position_ids, py::return_value_policy::reference_internal)
        .def("has_position_ids", &Request::has_position_ids)
        .def("mrope_last_pos", &Request::mrope_last_pos, py::return_value_policy::reference_internal)
        .def("has_mrope_last_pos", &Request::has_mrope_last_pos)
        .def("set_stop_token_ids", &Request::set_stop_token_ids, py::arg("stop_token_ids"))
        .def("stop_token_ids", &Request::stop_token_ids, py::return_value_policy::reference_internal)
        .def("set_ignore_stop_tokens", &Request::set_ignore_stop_tokens, py::arg("ignore") = true)
        .def("ignore_stop_tokens", &Request::ignore_stop_tokens);

    py::class_<Response>(m, "Response")
        .def(py::init<>())
        .def("token_ids", py::overload_cast<>(&Response::token_ids, py::const_), py::return_value_policy::reference_internal);

    py::class_<EdgeFM>(m, "EdgeFM")
        .def(py::init<const std::string&>(), py::arg("config_path"))
        .def("generate", &EdgeFM::generate, py::arg("request"), py::call_guard<py::gil_scoped_release>())
        .def("plan",
             [](const EdgeFM& self, int32_t request_id, const py::dict& inputs) {
                 TensorRefMap refs = tensor_ref_map_from_py_dict(inputs);
                 TensorMap result;
                 {
                     py::gil_scoped_release release;
                     result = self.plan(request_id, refs);
                 }
                 return tensor_map_to_py_dict(std::move(result));
             },
             py::arg("request_id"), py::arg("inputs"))
        .def("run_stage",
             [](const EdgeFM& self, int32_t request_id, const std::string& stage, const py::dict& inputs) {
                 TensorRefMap refs = tensor_ref_map_from_py_dict(inputs);
                 TensorMap result;
                 {
                     py::gil_scoped_release release;
                     result = self.run_stage(request_id, stage, refs);
                 }
                 return tensor_map_to_py_dict(std::move(result));
             },
             py::arg("request_id"), py::arg("stage_name"), py::arg("inputs"))
        .def("prefill",
             [](const EdgeFM& self, int32_t request_id, const py::dict& inputs) {
                 TensorRefMap refs = tensor_ref_map_from_py_dict(inputs);
                 TensorMap result;
                 {
                     py::gil_scoped_release release;
                     result = self.prefill(request_id, refs);
                 }
                 return tensor_map_to_py_dict(std::move(result));
             },
             py::arg("request_id"), py::arg("inputs"))
        .def("decode",
             [](const EdgeFM& self, int32_t request_id, const py::dict& inputs) {
                 TensorRefMap refs = tensor_ref_map_from_py_dict(inputs);
                 TensorMap result;
                 {
                     py::gil_scoped_release release;
                     result = self.decode(request_id, refs);
                 }
                 return tensor_map_to_py_dict(std::move(result));
             },
             py::arg("request_id"), py::arg("inputs"))
        .def("last_stage_metrics", &EdgeFM::last_stage_metrics)
        .def("last_plan_metrics", &EdgeFM::last_plan_metrics)
        .def("last_generate_metrics", &EdgeFM::last_generate_metrics)
        .def("backend_handle", [](const EdgeFM& e) { return reinterpret_cast<std::uintptr_t>(e.backend_handle()); },
             "address of the engine's efm_b200_ctx (0 for engines without one), for C-ABI companions such as the vision encoder")
        .def("tune", &EdgeFM::tune);
}
