// Bindings of the VMM classes; same Python surface as the reference's
// python-ext/src/py_cumem.rs:19-338 (typed in pplx_garden/native/cumem.pyi).
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include "../core/error.h"
#include "../cumem/cumem.h"
#include "py_util.h"

namespace py = pybind11;
using namespace pplx;

namespace {

struct PyExportHandle {
  CUMemExportData data;
};

std::shared_ptr<CUMemMapping> map_handle(const std::shared_ptr<CUAllocHandleBase>& h,
                                         const py::object& device) {
  return h->map(h, pplx_py::device_index(device, -1));
}

py::object mapping_to_tensor(const std::shared_ptr<CUMemMapping>& self, const py::tuple& shape,
                             const py::object& dtype) {
  PPLX_REQUIRE(self->mapped(), "the mapping was unmapped");
  uint64_t bytes = dtype.attr("itemsize").cast<uint64_t>();
  for (const auto& d : shape) bytes *= d.cast<uint64_t>();
  if (bytes > self->size()) {
    throw Error(ErrorKind::kInvalidArgument,
                "requested tensor of " + std::to_string(bytes) + " bytes exceeds the mapping of " +
                    std::to_string(self->size()) + " bytes");
  }
  py::object flat = pplx_py::device_bytes_tensor(self->data_ptr(), bytes, self->device_id(),
                                                 py::cast(self));
  return flat.attr("view")(dtype).attr("view")(shape);
}

}  // namespace

void bind_cumem(py::module_& m) {
  py::enum_<CUMemHandleKind>(m, "CUMemHandleKind")
      .value("Local", CUMemHandleKind::kLocal)
      .value("FileDescriptor", CUMemHandleKind::kFileDescriptor)
      .value("Fabric", CUMemHandleKind::kFabric);

  py::class_<CUMemMapping, std::shared_ptr<CUMemMapping>>(m, "CUMemMapping")
      .def_property_readonly("size", &CUMemMapping::size)
      .def_property_readonly("device_id", &CUMemMapping::device_id)
      .def("data_ptr", &CUMemMapping::data_ptr)
      .def("to_tensor", &mapping_to_tensor, py::arg("shape"), py::arg("dtype"))
      .def("unmap", &CUMemMapping::unmap);

  py::class_<CUAllocHandleBase, std::shared_ptr<CUAllocHandleBase>>(m, "CUAllocHandle")
      .def_property_readonly("size", &CUAllocHandleBase::size)
      .def("map", &map_handle, py::arg("device") = py::none())
      .def("map_to", [](const std::shared_ptr<CUAllocHandleBase>& self, CUMemMapping& mapping) {
        self->map_to(self, mapping);
      });

  py::class_<PyExportHandle>(m, "CUMemExportHandle")
      .def("bind",
           [](const PyExportHandle& self, const py::object& device) {
             int dev = pplx_py::device_index(device, -1);
             if (dev < 0) {
               PPLX_CUDA_CHECK(cudaGetDevice(&dev));
             }
             return std::make_shared<CUMemImportHandle>(self.data, dev);
           },
           py::arg("device") = py::none(),
           "Import the allocation into this process (for the current CUDA device by default).")
      .def_property_readonly("size", [](const PyExportHandle& s) { return s.data.size; })
      .def("as_bytes", [](const PyExportHandle& s) { return py::bytes(s.data.serialize()); })
      .def_static("from_bytes",
                  [](const py::bytes& b) { return PyExportHandle{CUMemExportData::deserialize(b)}; })
      .def(py::pickle([](const PyExportHandle& s) { return py::bytes(s.data.serialize()); },
                      [](const py::bytes& b) {
                        return PyExportHandle{CUMemExportData::deserialize(b)};
                      }));

  py::class_<CUMemImportHandle, CUAllocHandleBase, std::shared_ptr<CUMemImportHandle>>(
      m, "CUMemImportHandle");

  py::class_<CUMemAllocHandle, CUAllocHandleBase, std::shared_ptr<CUMemAllocHandle>>(
      m, "CUMemAllocHandle")
      .def(py::init([](size_t size, const py::object& device, CUMemHandleKind kind) {
             int dev = pplx_py::device_index(device, -1);
             if (dev < 0) PPLX_CUDA_CHECK(cudaGetDevice(&dev));
             return std::make_shared<CUMemAllocHandle>(size, dev, kind);
           }),
           py::arg("size"), py::arg("device"), py::arg("handle_kind") = CUMemHandleKind::kLocal)
      .def("export", [](CUMemAllocHandle& self) { return PyExportHandle{self.export_handle()}; });

  struct PyMcExport {
    CUMemExportData data;
  };
  py::class_<PyMcExport>(m, "CUMulticastExportHandle")
      .def("bind",
           [](const PyMcExport& self, const py::object& device) {
             int dev = pplx_py::device_index(device, -1);
             if (dev < 0) PPLX_CUDA_CHECK(cudaGetDevice(&dev));
             return std::make_shared<CUMulticastHandle>(self.data, dev);
           },
           py::arg("device") = py::none())
      .def(py::pickle([](const PyMcExport& s) { return py::bytes(s.data.serialize()); },
                      [](const py::bytes& b) { return PyMcExport{CUMemExportData::deserialize(b)}; }));

  py::class_<CUMulticastHandle, CUAllocHandleBase, std::shared_ptr<CUMulticastHandle>>(
      m, "CUMulticastHandle")
      .def(py::init([](int num_devices, size_t size, CUMemHandleKind kind) {
             return std::make_shared<CUMulticastHandle>(num_devices, size, kind);
           }),
           py::arg("num_devices"), py::arg("size"),
           py::arg("handle_kind") = CUMemHandleKind::kLocal)
      .def("export", [](CUMulticastHandle& self) { return PyMcExport{self.export_handle()}; })
      .def("add_device",
           [](CUMulticastHandle& self, const py::object& device) {
             self.add_device(pplx_py::device_index(device, 0));
           },
           py::arg("device_index"))
      .def("bind_mem", [](CUMulticastHandle& self, const CUMemAllocHandle& alloc) {
        self.bind_mem(alloc);
      })
      .def("unbind", [](CUMulticastHandle& self) { self.unbind(); },
           "Take this process's memory out of the multicast object (before freeing it or exiting).")
      .def_static("supported", [](const py::object& device) {
        return CUMulticastHandle::supported(pplx_py::device_index(device, 0));
      });

  // file-descriptor transport, exposed for tests
  m.def("_fd_server_name", &fd_server_name);
  m.def("_fd_server_register", &fd_server_register);
  m.def("_fd_server_unregister", &fd_server_unregister);
  m.def("_fd_fetch", &fd_fetch, py::arg("pid"), py::arg("fd"), py::arg("socket_name"));
  m.def("_fd_fetch_set_mode", &fd_fetch_set_mode);
}
