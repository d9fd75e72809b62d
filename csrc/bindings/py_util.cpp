#include "py_util.h"

#include <cuda_runtime.h>

#include "../core/error.h"

namespace pplx_py {

int device_index(const py::handle& obj, int fallback) {
  if (obj.is_none()) return fallback;
  if (py::isinstance<py::int_>(obj)) return obj.cast<int>();
  if (py::isinstance<py::str>(obj)) {
    const std::string s = obj.cast<std::string>();
    if (s == "cpu") return -1;
    if (s == "cuda") return fallback;
    if (s.rfind("cuda:", 0) == 0) return std::stoi(s.substr(5));
    throw pplx::Error(pplx::ErrorKind::kInvalidArgument, "cannot parse device string '" + s + "'");
  }
  if (py::hasattr(obj, "type")) {
    const std::string type = py::str(obj.attr("type"));
    if (type == "cpu") return -1;
    py::object index = obj.attr("index");
    if (index.is_none()) return fallback;
    return index.cast<int>();
  }
  throw pplx::Error(pplx::ErrorKind::kInvalidArgument, "expected a torch.device, str or int");
}

DtypeInfo dtype_info(const py::handle& dtype) {
  DtypeInfo info;
  info.name = py::str(dtype);
  info.itemsize = dtype.attr("itemsize").cast<int>();
  // codes follow c10::ScalarType
  if (info.name == "torch.float16") info.code = 5;
  else if (info.name == "torch.float32") info.code = 6;
  else if (info.name == "torch.bfloat16") info.code = 15;
  else if (info.name == "torch.float8_e4m3fn") info.code = 24;
  else if (info.name == "torch.float8_e5m2") info.code = 23;
  else if (info.name == "torch.uint8") info.code = 0;
  else if (info.name == "torch.int8") info.code = 1;
  else if (info.name == "torch.int32") info.code = 3;
  else if (info.name == "torch.int64") info.code = 4;
  else if (info.name == "torch.uint32") info.code = 28;
  else info.code = -1;
  return info;
}

namespace {

// DLPack ABI (v0.8 layout; stable).
struct DLDevice {
  int32_t device_type;
  int32_t device_id;
};
struct DLDataType {
  uint8_t code;
  uint8_t bits;
  uint16_t lanes;
};
struct DLTensor {
  void* data;
  DLDevice device;
  int32_t ndim;
  DLDataType dtype;
  int64_t* shape;
  int64_t* strides;
  uint64_t byte_offset;
};
struct DLManagedTensor {
  DLTensor dl_tensor;
  void* manager_ctx;
  void (*deleter)(DLManagedTensor*);
};

struct Holder {
  DLManagedTensor managed;
  int64_t shape[1];
  int64_t strides[1];
  PyObject* owner;
};

void holder_deleter(DLManagedTensor* t) {
  Holder* h = static_cast<Holder*>(t->manager_ctx);
  if (h->owner != nullptr) {
    py::gil_scoped_acquire gil;
    Py_DECREF(h->owner);
  }
  delete h;
}

void capsule_destructor(PyObject* capsule) {
  // Only called when nobody consumed the capsule (its name is still "dltensor").
  if (PyCapsule_IsValid(capsule, "dltensor")) {
    auto* t = static_cast<DLManagedTensor*>(PyCapsule_GetPointer(capsule, "dltensor"));
    if (t != nullptr && t->deleter != nullptr) t->deleter(t);
  }
}

}  // namespace

py::object device_bytes_capsule(uint64_t ptr, uint64_t nbytes, int device, py::object owner) {
  auto* h = new Holder();
  h->shape[0] = static_cast<int64_t>(nbytes);
  h->strides[0] = 1;
  h->owner = owner.is_none() ? nullptr : owner.release().ptr();
  DLTensor& t = h->managed.dl_tensor;
  t.data = reinterpret_cast<void*>(ptr);
  t.device = device >= 0 ? DLDevice{2 /* kDLCUDA */, device} : DLDevice{1 /* kDLCPU */, 0};
  t.ndim = 1;
  t.dtype = DLDataType{1 /* kDLUInt */, 8, 1};
  t.shape = h->shape;
  t.strides = h->strides;
  t.byte_offset = 0;
  h->managed.manager_ctx = h;
  h->managed.deleter = holder_deleter;
  PyObject* cap = PyCapsule_New(&h->managed, "dltensor", capsule_destructor);
  if (cap == nullptr) {
    holder_deleter(&h->managed);
    throw py::error_already_set();
  }
  return py::reinterpret_steal<py::object>(cap);
}

py::object device_bytes_tensor(uint64_t ptr, uint64_t nbytes, int device, py::object owner) {
  py::object capsule = device_bytes_capsule(ptr, nbytes, device, std::move(owner));
  py::object torch = py::module_::import("torch");
  return torch.attr("from_dlpack")(capsule);
}

namespace {
struct ProfilerHooks {
  py::object module;  // torch.autograd.profiler
  py::object enter;   // torch.ops.profiler._record_function_enter_new
  py::object exit;    // torch.ops.profiler._record_function_exit._RecordFunction
  bool ok = false;
};

ProfilerHooks& profiler_hooks() {
  // leaked on purpose: destroying Python objects after the interpreter is gone would crash
  static ProfilerHooks* hooks = [] {
    auto* h = new ProfilerHooks();
    try {
      h->module = py::module_::import("torch.autograd.profiler");
      py::object ops = py::module_::import("torch").attr("ops").attr("profiler");
      h->enter = ops.attr("_record_function_enter_new");
      h->exit = ops.attr("_record_function_exit").attr("_RecordFunction");
      h->ok = true;
    } catch (const py::error_already_set&) {
      h->ok = false;   // torch is not importable: ranges are simply not recorded
    }
    return h;
  }();
  return *hooks;
}
}  // namespace

TorchProfilerGuard::TorchProfilerGuard(const char* name) {
  ProfilerHooks& h = profiler_hooks();
  if (!h.ok) return;
  try {
    if (!h.module.attr("_is_profiler_enabled").cast<bool>()) return;
    handle_ = h.enter(py::str(name), py::none());
  } catch (const py::error_already_set&) {
    handle_ = py::object();
  }
}

TorchProfilerGuard::~TorchProfilerGuard() {
  if (!handle_) return;
  try {
    profiler_hooks().exit(handle_);
  } catch (const py::error_already_set&) {
    // a profiler that stopped in between: nothing to close
  }
}

}  // namespace pplx_py
