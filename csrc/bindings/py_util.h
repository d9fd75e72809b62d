// Helpers shared by the binding translation units.
#pragma once

#include <pybind11/pybind11.h>

#include <cstdint>
#include <string>

namespace pplx_py {

namespace py = pybind11;

// Accepts torch.device, "cuda:3", "cuda", an int or None (-> current device / fallback).
// Same inputs as the reference's PyDevice extractor (python-ext/src/py_device.rs:6-24).
int device_index(const py::handle& obj, int fallback = 0);

// torch.dtype -> (element size, scalar type code as in torch's ScalarType enum)
struct DtypeInfo {
  int itemsize;
  int code;
  std::string name;
};
DtypeInfo dtype_info(const py::handle& dtype);

// Zero-copy 1-D uint8 DLPack capsule over device memory; `owner` is kept alive until
// the consumer releases the tensor.
py::object device_bytes_capsule(uint64_t ptr, uint64_t nbytes, int device, py::object owner);

// torch tensor (uint8, 1-D) viewing [ptr, ptr+nbytes) on cuda:`device`.
py::object device_bytes_tensor(uint64_t ptr, uint64_t nbytes, int device, py::object owner);

// Scope that shows up in a torch profiler trace as a named range, opened from native code. The
// reference does the same with at::RecordFunction (rust/torch-lib/src/torch_lib.cc:121-130); this
// extension does not link libtorch, so it goes through torch's own operator pair
// profiler::_record_function_enter_new / _record_function_exit, and only while a profiler is
// running (one attribute read otherwise). Needs the GIL, which binding entry points hold.
class TorchProfilerGuard {
 public:
  explicit TorchProfilerGuard(const char* name);
  ~TorchProfilerGuard();
  TorchProfilerGuard(const TorchProfilerGuard&) = delete;
  TorchProfilerGuard& operator=(const TorchProfilerGuard&) = delete;

 private:
  py::object handle_;
};

}  // namespace pplx_py
