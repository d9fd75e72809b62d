#include "cu_driver.h"

#include <dlfcn.h>

#include <mutex>

#include "error.h"

namespace pplx {
namespace {

struct Loaded {
  void* lib = nullptr;
  CuDriver table{};
  std::string error;
};

Loaded& loaded() {
  static Loaded l;
  static std::once_flag once;
  std::call_once(once, [] {
    l.lib = dlopen("libcuda.so.1", RTLD_NOW | RTLD_GLOBAL);
    if (l.lib == nullptr) {
      const char* e = dlerror();
      l.error = e ? e : "dlopen(libcuda.so.1) failed";
      return;
    }
    bool missing_required = false;
    auto bind = [&](auto& slot, const char* name, bool required) {
      slot = reinterpret_cast<std::remove_reference_t<decltype(slot)>>(dlsym(l.lib, name));
      if (slot == nullptr && required) {
        missing_required = true;
        l.error += std::string(l.error.empty() ? "" : ", ") + name;
      }
    };
    CuDriver& t = l.table;
    bind(t.cuInit, "cuInit", true);
    bind(t.cuGetErrorString, "cuGetErrorString", true);
    bind(t.cuGetErrorName, "cuGetErrorName", true);
    bind(t.cuDeviceGet, "cuDeviceGet", true);
    bind(t.cuDeviceGetAttribute, "cuDeviceGetAttribute", true);
    bind(t.cuCtxGetCurrent, "cuCtxGetCurrent", true);
    bind(t.cuCtxSetCurrent, "cuCtxSetCurrent", true);
    bind(t.cuDevicePrimaryCtxRetain, "cuDevicePrimaryCtxRetain", true);
    bind(t.cuMemGetAllocationGranularity, "cuMemGetAllocationGranularity", true);
    bind(t.cuMemCreate, "cuMemCreate", true);
    bind(t.cuMemRelease, "cuMemRelease", true);
    bind(t.cuMemAddressReserve, "cuMemAddressReserve", true);
    bind(t.cuMemAddressFree, "cuMemAddressFree", true);
    bind(t.cuMemMap, "cuMemMap", true);
    bind(t.cuMemUnmap, "cuMemUnmap", true);
    bind(t.cuMemSetAccess, "cuMemSetAccess", true);
    bind(t.cuMemExportToShareableHandle, "cuMemExportToShareableHandle", true);
    bind(t.cuMemImportFromShareableHandle, "cuMemImportFromShareableHandle", true);
    bind(t.cuMemGetAddressRange, "cuMemGetAddressRange_v2", true);
    bind(t.cuMemRetainAllocationHandle, "cuMemRetainAllocationHandle", false);
    bind(t.cuMemGetHandleForAddressRange, "cuMemGetHandleForAddressRange", false);
    bind(t.cuTensorMapEncodeTiled, "cuTensorMapEncodeTiled", false);
    bind(t.cuMulticastCreate, "cuMulticastCreate", false);
    bind(t.cuMulticastAddDevice, "cuMulticastAddDevice", false);
    bind(t.cuMulticastBindMem, "cuMulticastBindMem", false);
    bind(t.cuMulticastUnbind, "cuMulticastUnbind", false);
    bind(t.cuMulticastGetGranularity, "cuMulticastGetGranularity", false);
    if (missing_required) {
      l.error = "libcuda.so.1 lacks: " + l.error;
      dlclose(l.lib);
      l.lib = nullptr;
      return;
    }
    const CUresult r = t.cuInit(0);
    if (r != CUDA_SUCCESS) {
      l.error = "cuInit failed with code " + std::to_string(static_cast<int>(r));
      l.lib = nullptr;
    }
  });
  return l;
}

}  // namespace

const CuDriver& CuDriver::get() {
  Loaded& l = loaded();
  if (l.lib == nullptr) {
    throw Error(ErrorKind::kCudaDriver, "CUDA driver unavailable: " + l.error);
  }
  return l.table;
}

bool CuDriver::available() { return loaded().lib != nullptr; }

std::string cu_error_string(CUresult r) {
  const char* name = nullptr;
  const char* desc = nullptr;
  if (CuDriver::available()) {
    CuDriver::get().cuGetErrorName(r, &name);
    CuDriver::get().cuGetErrorString(r, &desc);
  }
  return std::string(name ? name : "CUDA_ERROR_?") + " (" + (desc ? desc : "unknown") + ", code " +
         std::to_string(static_cast<int>(r)) + ")";
}

void cu_check(CUresult r, const char* expr, const char* file, int line) {
  if (r != CUDA_SUCCESS) {
    throw Error(ErrorKind::kCudaDriver, "CUDA driver error " + cu_error_string(r) + " in `" +
                                            expr + "` at " + file + ":" + std::to_string(line));
  }
}

void cu_ensure_context(int device) {
  // cudaSetDevice initialises the primary context and makes it current on this thread.
  (void)CuDriver::get();
  PPLX_CUDA_CHECK(cudaSetDevice(device));
}

}  // namespace pplx
