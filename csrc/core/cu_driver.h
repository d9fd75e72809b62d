// Lazily bound CUDA driver API. The native module must import on machines without a
// GPU driver (CPU-only test boxes), so libcuda is opened on first use instead of being
// linked. Covers what the reference reaches through its cuda-sys bindgen crate
// (rust/cuda-lib/cuda-sys, rust/cuda-lib/src/driver.rs:42-57).
#pragma once

#include <cuda.h>

#include <string>

namespace pplx {

struct CuDriver {
  CUresult (*cuInit)(unsigned int);
  CUresult (*cuGetErrorString)(CUresult, const char**);
  CUresult (*cuGetErrorName)(CUresult, const char**);
  CUresult (*cuDeviceGet)(CUdevice*, int);
  CUresult (*cuDeviceGetAttribute)(int*, CUdevice_attribute, CUdevice);
  CUresult (*cuCtxGetCurrent)(CUcontext*);
  CUresult (*cuCtxSetCurrent)(CUcontext);
  CUresult (*cuDevicePrimaryCtxRetain)(CUcontext*, CUdevice);
  CUresult (*cuMemGetAllocationGranularity)(size_t*, const CUmemAllocationProp*,
                                            CUmemAllocationGranularity_flags);
  CUresult (*cuMemCreate)(CUmemGenericAllocationHandle*, size_t, const CUmemAllocationProp*,
                          unsigned long long);
  CUresult (*cuMemRelease)(CUmemGenericAllocationHandle);
  CUresult (*cuMemAddressReserve)(CUdeviceptr*, size_t, size_t, CUdeviceptr, unsigned long long);
  CUresult (*cuMemAddressFree)(CUdeviceptr, size_t);
  CUresult (*cuMemMap)(CUdeviceptr, size_t, size_t, CUmemGenericAllocationHandle,
                       unsigned long long);
  CUresult (*cuMemUnmap)(CUdeviceptr, size_t);
  CUresult (*cuMemSetAccess)(CUdeviceptr, size_t, const CUmemAccessDesc*, size_t);
  CUresult (*cuMemExportToShareableHandle)(void*, CUmemGenericAllocationHandle,
                                           CUmemAllocationHandleType, unsigned long long);
  CUresult (*cuMemImportFromShareableHandle)(CUmemGenericAllocationHandle*, void*,
                                             CUmemAllocationHandleType);
  CUresult (*cuMemGetAddressRange)(CUdeviceptr*, size_t*, CUdeviceptr);
  CUresult (*cuMemRetainAllocationHandle)(CUmemGenericAllocationHandle*, void*);
  CUresult (*cuMemGetHandleForAddressRange)(void*, CUdeviceptr, size_t,
                                            CUmemRangeHandleType, unsigned long long);
  CUresult (*cuTensorMapEncodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                     const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                     CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                     CUtensorMapFloatOOBfill);
  CUresult (*cuMulticastCreate)(CUmemGenericAllocationHandle*, const CUmulticastObjectProp*);
  CUresult (*cuMulticastAddDevice)(CUmemGenericAllocationHandle, CUdevice);
  CUresult (*cuMulticastBindMem)(CUmemGenericAllocationHandle, size_t,
                                 CUmemGenericAllocationHandle, size_t, size_t,
                                 unsigned long long);
  CUresult (*cuMulticastUnbind)(CUmemGenericAllocationHandle, CUdevice, size_t, size_t);
  CUresult (*cuMulticastGetGranularity)(size_t*, const CUmulticastObjectProp*,
                                        CUmulticastGranularity_flags);

  // Throws pplx::Error(kCudaDriver) when libcuda cannot be opened.
  static const CuDriver& get();
  // True when libcuda.so.1 can be opened on this machine.
  static bool available();
};

void cu_check(CUresult r, const char* expr, const char* file, int line);
std::string cu_error_string(CUresult r);

#define PPLX_CU_CHECK(expr) ::pplx::cu_check((expr), #expr, __FILE__, __LINE__)

// Makes the primary context of `device` current on the calling thread.
void cu_ensure_context(int device);

}  // namespace pplx
