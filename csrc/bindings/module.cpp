// Python extension `pplx_garden._native` (also importable as `pplx_garden._rust`, the
// module name the reference's PyO3 extension uses: python-ext/src/lib.rs:8-21).
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include "../core/cu_driver.h"
#include "../core/error.h"
#include "../core/log.h"
#include "../core/thread_util.h"
#include "py_util.h"

namespace py = pybind11;

void bind_cumem(py::module_& m);
void bind_a2a(py::module_& m);
void bind_fabric(py::module_& m);
void bind_unigram(py::module_& m);
void bind_ops(py::module_& m);

PYBIND11_MODULE(_native, m) {
  m.doc() = "pplx_garden native core (C++/CUDA, sm_100a)";
  pplx::log_init_from_env();

  py::register_exception_translator([](std::exception_ptr p) {
    try {
      if (p) std::rethrow_exception(p);
    } catch (const pplx::Error& e) {
      switch (e.kind()) {
        case pplx::ErrorKind::kInvalidArgument:
          PyErr_SetString(PyExc_ValueError, e.what());
          break;
        case pplx::ErrorKind::kTimeout:
          PyErr_SetString(PyExc_TimeoutError, e.what());
          break;
        default:
          PyErr_SetString(PyExc_RuntimeError, e.what());
      }
    }
  });

  m.def("cuda_driver_available", [] { return pplx::CuDriver::available(); },
        "True when libcuda.so.1 can be loaded in this process.");
  m.def(
      "_profiler_guard_probe",
      [](const std::string& name) {
        bool enabled = false;
        try {
          enabled = py::module_::import("torch.autograd.profiler").attr("_is_profiler_enabled").cast<bool>();
        } catch (const py::error_already_set&) {
          enabled = false;
        }
        pplx_py::TorchProfilerGuard guard(name.c_str());
        return enabled;
      },
      py::arg("name"), "Opens and closes one native profiler range; returns whether a profiler was running.");
  m.def("pin_cpu", &pplx::pin_cpu, py::arg("cpu"), "Pin the calling thread to one logical CPU.");
  m.def("current_affinity", &pplx::current_affinity);
  m.def("log_set_level", [](const std::string& level) {
    if (level == "error") pplx::log_set_level(pplx::LogLevel::kError);
    else if (level == "warn") pplx::log_set_level(pplx::LogLevel::kWarn);
    else if (level == "info") pplx::log_set_level(pplx::LogLevel::kInfo);
    else if (level == "debug") pplx::log_set_level(pplx::LogLevel::kDebug);
    else if (level == "trace") pplx::log_set_level(pplx::LogLevel::kTrace);
    else throw pplx::Error(pplx::ErrorKind::kInvalidArgument, "unknown log level " + level);
  });
  m.def("log_render",
        [](const std::string& level, const std::string& target, const std::string& msg, bool json,
           bool color, double unix_time) {
          pplx::LogLevel l = pplx::LogLevel::kInfo;
          if (level == "error") l = pplx::LogLevel::kError;
          else if (level == "warn") l = pplx::LogLevel::kWarn;
          else if (level == "debug") l = pplx::LogLevel::kDebug;
          else if (level == "trace") l = pplx::LogLevel::kTrace;
          return pplx::log_render(l, target.c_str(), msg,
                                  json ? pplx::LogFormat::kJson : pplx::LogFormat::kText, color,
                                  unix_time);
        });
  m.def("log_message", [](const std::string& level, const std::string& target, const std::string& msg) {
    pplx::LogLevel l = pplx::LogLevel::kInfo;
    if (level == "error") l = pplx::LogLevel::kError;
    else if (level == "warn") l = pplx::LogLevel::kWarn;
    else if (level == "debug") l = pplx::LogLevel::kDebug;
    if (pplx::log_enabled(l)) pplx::log_message(l, target.c_str(), "%s", msg.c_str());
  });

  m.def("_tensor_from_ptr",
        [](uint64_t ptr, uint64_t nbytes, int device) {
          return pplx_py::device_bytes_tensor(ptr, nbytes, device, py::none());
        },
        py::arg("ptr"), py::arg("nbytes"), py::arg("device"),
        "uint8 tensor over raw memory the caller keeps alive (device >= 0: CUDA, -1: host).");

  bind_cumem(m);
  bind_a2a(m);
  bind_fabric(m);
  bind_unigram(m);
  bind_ops(m);
}
