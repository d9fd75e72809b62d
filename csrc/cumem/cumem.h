// CUDA virtual-memory-management allocations that can be shared between the processes
// of one node and mapped by every GPU of an NVLink domain, plus NVLS multicast objects.
//
// Same capabilities as the reference's rust/cuda-lib/src/cumem.rs:54-634
// (CUMemAllocHandle / CUMemMapping / export+import / CUMulticastHandle). Differences:
//   * a POSIX file descriptor is handed to the importer either with pidfd_getfd (as the
//     reference does, needs ptrace permission over the exporter) or, when that is not
//     permitted, over a per-process unix socket with SCM_RIGHTS;
//   * handles are reference counted with shared_ptr, mappings keep their allocation alive.
#pragma once

#include <cuda.h>

#include <array>
#include <cstdint>
#include <memory>
#include <string>
#include <vector>

namespace pplx {

enum class CUMemHandleKind : int { kLocal = 0, kFileDescriptor = 1, kFabric = 2 };

class CUMemMapping;

// Anything that owns a CUmemGenericAllocationHandle and can be mapped.
class CUAllocHandleBase {
 public:
  virtual ~CUAllocHandleBase();
  CUmemGenericAllocationHandle raw() const { return handle_; }
  size_t size() const { return size_; }
  // Reserves address space on `device` (default: the owning device), maps the
  // allocation there and grants that device read/write access.
  std::shared_ptr<CUMemMapping> map(std::shared_ptr<CUAllocHandleBase> self, int device = -1);
  // Replaces what `mapping` points at with this allocation (same size required).
  void map_to(std::shared_ptr<CUAllocHandleBase> self, CUMemMapping& mapping);
  int device() const { return device_; }

 protected:
  CUAllocHandleBase() = default;
  CUmemGenericAllocationHandle handle_ = 0;
  size_t size_ = 0;
  int device_ = 0;
  bool released_ = false;
};

class CUMemMapping {
 public:
  CUMemMapping(std::shared_ptr<CUAllocHandleBase> alloc, CUdeviceptr va, size_t size, int device);
  ~CUMemMapping();
  CUMemMapping(const CUMemMapping&) = delete;
  CUMemMapping& operator=(const CUMemMapping&) = delete;

  size_t size() const { return size_; }
  uint64_t data_ptr() const { return static_cast<uint64_t>(va_); }
  int device_id() const { return device_; }
  void unmap();
  bool mapped() const { return mapped_; }

 private:
  friend class CUAllocHandleBase;
  std::shared_ptr<CUAllocHandleBase> alloc_;
  CUdeviceptr va_;
  size_t size_;
  int device_;
  bool mapped_ = true;
};

// What travels to another process (picklable plain data).
struct CUMemExportData {
  CUMemHandleKind kind = CUMemHandleKind::kLocal;
  uint64_t size = 0;
  int32_t device = 0;          // owner's device ordinal (informational)
  int32_t pid = 0;             // exporter process
  int32_t fd = -1;             // fd number inside the exporter
  std::string socket_name;     // abstract unix socket of the exporter's fd server
  std::array<uint8_t, 64> fabric{};  // CUmemFabricHandle
  bool multicast = false;
  int32_t num_devices = 0;     // multicast only

  std::string serialize() const;
  static CUMemExportData deserialize(const std::string& bytes);
};

class CUMemImportHandle : public CUAllocHandleBase {
 public:
  // `device` is the importing process's GPU (where map() maps by default).
  CUMemImportHandle(const CUMemExportData& data, int device);
};

class CUMemAllocHandle : public CUAllocHandleBase {
 public:
  // Physical allocation on `device`, rounded up to the allocation granularity,
  // created as GPUDirect-RDMA capable where the device supports it.
  CUMemAllocHandle(size_t size, int device, CUMemHandleKind kind);
  ~CUMemAllocHandle() override;
  CUMemHandleKind kind() const { return kind_; }
  size_t requested_size() const { return requested_; }
  CUMemExportData export_handle();

 private:
  CUMemHandleKind kind_;
  size_t requested_;
  int exported_fd_ = -1;
};

class CUMulticastHandle : public CUAllocHandleBase {
 public:
  CUMulticastHandle(int num_devices, size_t size, CUMemHandleKind kind);
  CUMulticastHandle(const CUMemExportData& data, int device);  // import
  ~CUMulticastHandle() override;
  void add_device(int device);
  void bind_mem(const CUAllocHandleBase& alloc);
  // Takes this process's device memory out of the multicast object again. Every process unbinds
  // before it frees the bound allocation or exits; the destructor does it if the caller forgot.
  void unbind();
  CUMemExportData export_handle();
  int num_devices() const { return num_devices_; }
  // True when the driver and device expose multicast objects.
  static bool supported(int device);

 private:
  CUMemHandleKind kind_;
  int num_devices_;
  int exported_fd_ = -1;
  size_t bound_bytes_ = 0;   // bytes of this process's memory bound at offset 0
  int bound_device_ = -1;
};

// Rounds `size` up to the minimum allocation granularity of `device`.
size_t cumem_granularity(int device, CUMemHandleKind kind);

// ---- file-descriptor transport (exposed for tests; no GPU needed) ----

// Starts (once) the thread that serves this process's registered descriptors and
// returns the abstract socket name peers connect to.
std::string fd_server_name();
void fd_server_register(int fd);
void fd_server_unregister(int fd);
// Obtains a duplicate of descriptor `fd` of process `pid`: dup() inside one process,
// else pidfd_getfd, else the exporter's socket. Throws pplx::Error.
int fd_fetch(int pid, int fd, const std::string& socket_name);
// Forces one transport for tests: "auto", "pidfd" or "socket".
void fd_fetch_set_mode(const std::string& mode);

}  // namespace pplx
