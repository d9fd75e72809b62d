#include "cumem.h"

#include <fcntl.h>
#include <poll.h>
#include <sys/eventfd.h>
#include <sys/socket.h>
#include <sys/syscall.h>
#include <sys/un.h>
#include <unistd.h>

#include <atomic>
#include <cstring>
#include <mutex>
#include <random>
#include <set>
#include <thread>

#include "../core/cu_driver.h"
#include "../core/error.h"
#define PPLX_LOG_TARGET "pplx_garden::cumem"
#include "../core/log.h"

namespace pplx {

// ---------------------------------------------------------------------------
// file-descriptor transport
// ---------------------------------------------------------------------------
namespace {

#ifndef SYS_pidfd_open
#define SYS_pidfd_open 434
#endif
#ifndef SYS_pidfd_getfd
#define SYS_pidfd_getfd 438
#endif

struct FdServer {
  std::mutex mu;
  std::set<int> fds;
  std::string name;    // bound (abstract) socket name; visible to every local user
  uint64_t token = 0;  // secret of this process: travels only inside export handles
  int listen_fd = -1;
  int stop_fd = -1;
  std::thread thread;
  bool started = false;

  ~FdServer() {
    if (started) {
      uint64_t one = 1;
      (void)!write(stop_fd, &one, sizeof(one));
      if (thread.joinable()) thread.join();
      close(listen_fd);
      close(stop_fd);
    }
  }

  static socklen_t make_addr(const std::string& nm, sockaddr_un* addr) {
    std::memset(addr, 0, sizeof(*addr));
    addr->sun_family = AF_UNIX;
    // abstract namespace: leading NUL, no filesystem entry to clean up
    const size_t n = std::min(nm.size(), sizeof(addr->sun_path) - 2);
    std::memcpy(addr->sun_path + 1, nm.data(), n);
    return static_cast<socklen_t>(offsetof(sockaddr_un, sun_path) + 1 + n);
  }

  void start() {
    std::lock_guard<std::mutex> lock(mu);
    if (started) return;
    std::random_device rd;
    name = "pplx-cumem-" + std::to_string(getpid()) + "-" + std::to_string(rd());
    token = (static_cast<uint64_t>(rd()) << 32) ^ rd();
    listen_fd = socket(AF_UNIX, SOCK_STREAM | SOCK_CLOEXEC, 0);
    if (listen_fd < 0) throw Error::from_errno("socket(AF_UNIX)");
    sockaddr_un addr;
    const socklen_t len = make_addr(name, &addr);
    if (bind(listen_fd, reinterpret_cast<sockaddr*>(&addr), len) != 0) {
      const int e = errno;
      close(listen_fd);
      throw Error::from_errno("bind(fd server)", e);
    }
    if (listen(listen_fd, 64) != 0) {
      const int e = errno;
      close(listen_fd);
      throw Error::from_errno("listen(fd server)", e);
    }
    stop_fd = eventfd(0, EFD_CLOEXEC);
    thread = std::thread([this] { loop(); });
    started = true;
  }

  // The name of an abstract socket can be read from /proc/net/unix by any local user, so a
  // connection proves nothing. A descriptor is handed out only to a peer that runs under this
  // process's user id (SO_PEERCRED, filled in by the kernel) and that presents the token carried
  // by the export handle; everybody else gets payload 0 and no descriptor.
  void serve_one(int conn) {
    struct Request {
      int32_t wanted;
      uint32_t pad;
      uint64_t token;
    } req{-1, 0, 0};
    if (recv(conn, &req, sizeof(req), MSG_WAITALL) != sizeof(req)) return;
    const int32_t wanted = req.wanted;
    ucred cred{};
    socklen_t cred_len = sizeof(cred);
    const bool same_user = getsockopt(conn, SOL_SOCKET, SO_PEERCRED, &cred, &cred_len) == 0 &&
                           cred.uid == geteuid();
    bool known;
    {
      std::lock_guard<std::mutex> lock(mu);
      known = same_user && req.token == token && fds.count(wanted) != 0;
    }
    char payload = known ? 1 : 0;
    iovec iov{&payload, 1};
    msghdr msg{};
    msg.msg_iov = &iov;
    msg.msg_iovlen = 1;
    alignas(cmsghdr) char control[CMSG_SPACE(sizeof(int))];
    if (known) {
      std::memset(control, 0, sizeof(control));
      msg.msg_control = control;
      msg.msg_controllen = sizeof(control);
      cmsghdr* c = CMSG_FIRSTHDR(&msg);
      c->cmsg_level = SOL_SOCKET;
      c->cmsg_type = SCM_RIGHTS;
      c->cmsg_len = CMSG_LEN(sizeof(int));
      std::memcpy(CMSG_DATA(c), &wanted, sizeof(int));
    }
    (void)!sendmsg(conn, &msg, MSG_NOSIGNAL);
  }

  void loop() {
    for (;;) {
      pollfd p[2] = {{listen_fd, POLLIN, 0}, {stop_fd, POLLIN, 0}};
      const int rc = poll(p, 2, -1);
      if (rc < 0) {
        if (errno == EINTR) continue;
        return;
      }
      if (p[1].revents & POLLIN) return;
      if (p[0].revents & POLLIN) {
        const int conn = accept4(listen_fd, nullptr, nullptr, SOCK_CLOEXEC);
        if (conn < 0) continue;
        timeval tv{2, 0};
        setsockopt(conn, SOL_SOCKET, SO_RCVTIMEO, &tv, sizeof(tv));
        serve_one(conn);
        close(conn);
      }
    }
  }
};

FdServer& fd_server() {
  static FdServer* s = new FdServer();  // leaked on purpose: outlives static destructors
  return *s;
}

std::atomic<int> g_fetch_mode{0};  // 0 auto, 1 pidfd, 2 socket

int fetch_by_pidfd(int pid, int fd) {
  const int pidfd = static_cast<int>(syscall(SYS_pidfd_open, pid, 0));
  if (pidfd < 0) return -errno;
  const int got = static_cast<int>(syscall(SYS_pidfd_getfd, pidfd, fd, 0));
  const int err = errno;
  close(pidfd);
  return got < 0 ? -err : got;
}

int fetch_by_socket(int fd, const std::string& name_and_token) {
  // "<socket name>:<token in hex>", as fd_server_name() returns it
  const size_t colon = name_and_token.rfind(':');
  const std::string socket_name = name_and_token.substr(0, colon);
  uint64_t token = 0;
  if (colon != std::string::npos) token = std::strtoull(name_and_token.c_str() + colon + 1, nullptr, 16);
  const int s = socket(AF_UNIX, SOCK_STREAM | SOCK_CLOEXEC, 0);
  if (s < 0) return -errno;
  sockaddr_un addr;
  const socklen_t len = FdServer::make_addr(socket_name, &addr);
  timeval tv{10, 0};
  setsockopt(s, SOL_SOCKET, SO_RCVTIMEO, &tv, sizeof(tv));
  setsockopt(s, SOL_SOCKET, SO_SNDTIMEO, &tv, sizeof(tv));
  if (connect(s, reinterpret_cast<sockaddr*>(&addr), len) != 0) {
    const int e = errno;
    close(s);
    return -e;
  }
  struct Request {
    int32_t wanted;
    uint32_t pad;
    uint64_t token;
  } wanted{fd, 0, token};
  if (send(s, &wanted, sizeof(wanted), MSG_NOSIGNAL) != sizeof(wanted)) {
    const int e = errno;
    close(s);
    return -e;
  }
  char payload = 0;
  iovec iov{&payload, 1};
  msghdr msg{};
  msg.msg_iov = &iov;
  msg.msg_iovlen = 1;
  alignas(cmsghdr) char control[CMSG_SPACE(sizeof(int))];
  msg.msg_control = control;
  msg.msg_controllen = sizeof(control);
  const ssize_t n = recvmsg(s, &msg, MSG_CMSG_CLOEXEC);
  const int e = errno;
  close(s);
  if (n != 1) return n < 0 ? -e : -EPROTO;
  if (payload != 1) return -EBADF;
  for (cmsghdr* c = CMSG_FIRSTHDR(&msg); c != nullptr; c = CMSG_NXTHDR(&msg, c)) {
    if (c->cmsg_level == SOL_SOCKET && c->cmsg_type == SCM_RIGHTS) {
      int got;
      std::memcpy(&got, CMSG_DATA(c), sizeof(int));
      return got;
    }
  }
  return -EPROTO;
}

}  // namespace

std::string fd_server_name() {
  fd_server().start();
  char hex[32];
  std::snprintf(hex, sizeof(hex), ":%016llx", static_cast<unsigned long long>(fd_server().token));
  return fd_server().name + hex;
}

void fd_server_register(int fd) {
  fd_server().start();
  std::lock_guard<std::mutex> lock(fd_server().mu);
  fd_server().fds.insert(fd);
}

void fd_server_unregister(int fd) {
  std::lock_guard<std::mutex> lock(fd_server().mu);
  fd_server().fds.erase(fd);
}

void fd_fetch_set_mode(const std::string& mode) {
  if (mode == "auto") g_fetch_mode = 0;
  else if (mode == "pidfd") g_fetch_mode = 1;
  else if (mode == "socket") g_fetch_mode = 2;
  else throw Error(ErrorKind::kInvalidArgument, "fd_fetch_set_mode: unknown mode " + mode);
}

int fd_fetch(int pid, int fd, const std::string& socket_name) {
  const int mode = g_fetch_mode.load();
  if (pid == getpid() && mode == 0) {
    const int d = fcntl(fd, F_DUPFD_CLOEXEC, 0);
    if (d < 0) throw Error::from_errno("dup(exported fd)");
    return d;
  }
  int pidfd_err = 0;
  if (mode != 2) {
    const int got = fetch_by_pidfd(pid, fd);
    if (got >= 0) return got;
    pidfd_err = -got;
    if (mode == 1) throw Error::from_errno("pidfd_getfd(pid " + std::to_string(pid) + ")", pidfd_err);
  }
  if (socket_name.empty()) {
    throw Error::from_errno("pidfd_getfd failed and the exporter runs no fd server", pidfd_err);
  }
  const int got = fetch_by_socket(fd, socket_name);
  if (got >= 0) return got;
  throw Error::from_errno("receiving fd " + std::to_string(fd) + " of pid " + std::to_string(pid) +
                              " over @" + socket_name +
                              (pidfd_err ? " (pidfd_getfd: " + std::string(std::strerror(pidfd_err)) + ")" : ""),
                          -got);
}

// ---------------------------------------------------------------------------
// export data (de)serialisation: a tiny tagged little-endian format
// ---------------------------------------------------------------------------

namespace {
void put_u32(std::string* s, uint32_t v) { s->append(reinterpret_cast<const char*>(&v), 4); }
void put_u64(std::string* s, uint64_t v) { s->append(reinterpret_cast<const char*>(&v), 8); }
uint32_t get_u32(const std::string& s, size_t* off) {
  if (*off + 4 > s.size()) throw Error(ErrorKind::kInvalidArgument, "truncated export handle");
  uint32_t v;
  std::memcpy(&v, s.data() + *off, 4);
  *off += 4;
  return v;
}
uint64_t get_u64(const std::string& s, size_t* off) {
  if (*off + 8 > s.size()) throw Error(ErrorKind::kInvalidArgument, "truncated export handle");
  uint64_t v;
  std::memcpy(&v, s.data() + *off, 8);
  *off += 8;
  return v;
}
constexpr uint32_t kExportMagic = 0x4d454d43;  // "CMEM"
}  // namespace

std::string CUMemExportData::serialize() const {
  std::string s;
  put_u32(&s, kExportMagic);
  put_u32(&s, static_cast<uint32_t>(kind));
  put_u64(&s, size);
  put_u32(&s, static_cast<uint32_t>(device));
  put_u32(&s, static_cast<uint32_t>(pid));
  put_u32(&s, static_cast<uint32_t>(fd));
  put_u32(&s, multicast ? 1u : 0u);
  put_u32(&s, static_cast<uint32_t>(num_devices));
  put_u32(&s, static_cast<uint32_t>(socket_name.size()));
  s.append(socket_name);
  s.append(reinterpret_cast<const char*>(fabric.data()), fabric.size());
  return s;
}

CUMemExportData CUMemExportData::deserialize(const std::string& bytes) {
  size_t off = 0;
  if (get_u32(bytes, &off) != kExportMagic) {
    throw Error(ErrorKind::kInvalidArgument, "not a cumem export handle");
  }
  CUMemExportData d;
  d.kind = static_cast<CUMemHandleKind>(get_u32(bytes, &off));
  d.size = get_u64(bytes, &off);
  d.device = static_cast<int32_t>(get_u32(bytes, &off));
  d.pid = static_cast<int32_t>(get_u32(bytes, &off));
  d.fd = static_cast<int32_t>(get_u32(bytes, &off));
  d.multicast = get_u32(bytes, &off) != 0;
  d.num_devices = static_cast<int32_t>(get_u32(bytes, &off));
  const uint32_t n = get_u32(bytes, &off);
  if (off + n + d.fabric.size() > bytes.size()) {
    throw Error(ErrorKind::kInvalidArgument, "truncated export handle");
  }
  d.socket_name.assign(bytes.data() + off, n);
  off += n;
  std::memcpy(d.fabric.data(), bytes.data() + off, d.fabric.size());
  return d;
}

// ---------------------------------------------------------------------------
// allocations and mappings
// ---------------------------------------------------------------------------

namespace {

CUmemAllocationHandleType cu_handle_type(CUMemHandleKind kind) {
  switch (kind) {
    case CUMemHandleKind::kFileDescriptor: return CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
    case CUMemHandleKind::kFabric: return CU_MEM_HANDLE_TYPE_FABRIC;
    default: return CU_MEM_HANDLE_TYPE_NONE;
  }
}

CUmemAllocationProp alloc_prop(int device, CUMemHandleKind kind, bool rdma) {
  CUmemAllocationProp prop{};
  prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
  prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  prop.location.id = device;
  prop.requestedHandleTypes = cu_handle_type(kind);
  prop.allocFlags.gpuDirectRDMACapable = rdma ? 1 : 0;
  return prop;
}

bool device_supports_rdma(int device) {
  const CuDriver& cu = CuDriver::get();
  CUdevice dev;
  if (cu.cuDeviceGet(&dev, device) != CUDA_SUCCESS) return false;
  int v = 0;
  if (cu.cuDeviceGetAttribute(&v, CU_DEVICE_ATTRIBUTE_GPU_DIRECT_RDMA_WITH_CUDA_VMM_SUPPORTED,
                              dev) != CUDA_SUCCESS) {
    return false;
  }
  return v != 0;
}

}  // namespace

size_t cumem_granularity(int device, CUMemHandleKind kind) {
  const CuDriver& cu = CuDriver::get();
  const CUmemAllocationProp prop = alloc_prop(device, kind, false);
  size_t g = 0;
  PPLX_CU_CHECK(cu.cuMemGetAllocationGranularity(&g, &prop, CU_MEM_ALLOC_GRANULARITY_MINIMUM));
  return g;
}

CUAllocHandleBase::~CUAllocHandleBase() {
  if (handle_ != 0 && !released_ && CuDriver::available()) {
    CuDriver::get().cuMemRelease(handle_);
  }
}

std::shared_ptr<CUMemMapping> CUAllocHandleBase::map(std::shared_ptr<CUAllocHandleBase> self,
                                                     int device) {
  const CuDriver& cu = CuDriver::get();
  if (device < 0) device = device_;
  cu_ensure_context(device);
  CUdeviceptr va = 0;
  PPLX_CU_CHECK(cu.cuMemAddressReserve(&va, size_, 0, 0, 0));
  CUresult r = cu.cuMemMap(va, size_, 0, handle_, 0);
  if (r != CUDA_SUCCESS) {
    cu.cuMemAddressFree(va, size_);
    cu_check(r, "cuMemMap", __FILE__, __LINE__);
  }
  CUmemAccessDesc access{};
  access.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  access.location.id = device;
  access.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  r = cu.cuMemSetAccess(va, size_, &access, 1);
  if (r != CUDA_SUCCESS) {
    cu.cuMemUnmap(va, size_);
    cu.cuMemAddressFree(va, size_);
    cu_check(r, "cuMemSetAccess", __FILE__, __LINE__);
  }
  return std::make_shared<CUMemMapping>(std::move(self), va, size_, device);
}

void CUAllocHandleBase::map_to(std::shared_ptr<CUAllocHandleBase> self, CUMemMapping& mapping) {
  const CuDriver& cu = CuDriver::get();
  PPLX_REQUIRE(mapping.size_ == size_, "map_to: the mapping and the allocation differ in size");
  cu_ensure_context(mapping.device_);
  if (mapping.mapped_) {
    PPLX_CU_CHECK(cu.cuMemUnmap(mapping.va_, mapping.size_));
    mapping.mapped_ = false;
  }
  PPLX_CU_CHECK(cu.cuMemMap(mapping.va_, size_, 0, handle_, 0));
  CUmemAccessDesc access{};
  access.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  access.location.id = mapping.device_;
  access.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  PPLX_CU_CHECK(cu.cuMemSetAccess(mapping.va_, size_, &access, 1));
  mapping.alloc_ = std::move(self);
  mapping.mapped_ = true;
}

CUMemMapping::CUMemMapping(std::shared_ptr<CUAllocHandleBase> alloc, CUdeviceptr va, size_t size,
                           int device)
    : alloc_(std::move(alloc)), va_(va), size_(size), device_(device) {}

void CUMemMapping::unmap() {
  if (va_ == 0) return;
  if (CuDriver::available()) {
    const CuDriver& cu = CuDriver::get();
    if (mapped_) cu.cuMemUnmap(va_, size_);
    cu.cuMemAddressFree(va_, size_);
  }
  mapped_ = false;
  va_ = 0;
  alloc_.reset();
}

CUMemMapping::~CUMemMapping() { unmap(); }

CUMemAllocHandle::CUMemAllocHandle(size_t size, int device, CUMemHandleKind kind)
    : kind_(kind), requested_(size) {
  const CuDriver& cu = CuDriver::get();
  PPLX_REQUIRE(size > 0, "CUMemAllocHandle: size must be positive");
  cu_ensure_context(device);
  device_ = device;
  const size_t gran = cumem_granularity(device, kind);
  size_ = (size + gran - 1) / gran * gran;
  CUmemAllocationProp prop = alloc_prop(device, kind, device_supports_rdma(device));
  CUresult r = cu.cuMemCreate(&handle_, size_, &prop, 0);
  if (r != CUDA_SUCCESS && prop.allocFlags.gpuDirectRDMACapable) {
    prop.allocFlags.gpuDirectRDMACapable = 0;
    r = cu.cuMemCreate(&handle_, size_, &prop, 0);
  }
  cu_check(r, "cuMemCreate", __FILE__, __LINE__);
}

CUMemAllocHandle::~CUMemAllocHandle() {
  if (exported_fd_ >= 0) {
    fd_server_unregister(exported_fd_);
    close(exported_fd_);
  }
}

CUMemExportData CUMemAllocHandle::export_handle() {
  const CuDriver& cu = CuDriver::get();
  CUMemExportData d;
  d.kind = kind_;
  d.size = size_;
  d.device = device_;
  d.pid = getpid();
  switch (kind_) {
    case CUMemHandleKind::kFileDescriptor: {
      if (exported_fd_ < 0) {
        int fd = -1;
        PPLX_CU_CHECK(cu.cuMemExportToShareableHandle(
            &fd, handle_, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0));
        exported_fd_ = fd;
        fd_server_register(fd);
      }
      d.fd = exported_fd_;
      d.socket_name = fd_server_name();
      break;
    }
    case CUMemHandleKind::kFabric: {
      CUmemFabricHandle fh;
      PPLX_CU_CHECK(cu.cuMemExportToShareableHandle(&fh, handle_, CU_MEM_HANDLE_TYPE_FABRIC, 0));
      static_assert(sizeof(fh) == 64, "fabric handle is 64 bytes");
      std::memcpy(d.fabric.data(), &fh, sizeof(fh));
      break;
    }
    default:
      throw Error(ErrorKind::kInvalidArgument,
                  "a Local allocation cannot be exported; create it with FileDescriptor or Fabric");
  }
  return d;
}

namespace {
CUmemGenericAllocationHandle import_generic(const CUMemExportData& data) {
  const CuDriver& cu = CuDriver::get();
  CUmemGenericAllocationHandle h = 0;
  switch (data.kind) {
    case CUMemHandleKind::kFileDescriptor: {
      const int fd = fd_fetch(data.pid, data.fd, data.socket_name);
      const CUresult r = cu.cuMemImportFromShareableHandle(
          &h, reinterpret_cast<void*>(static_cast<uintptr_t>(fd)),
          CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR);
      close(fd);
      cu_check(r, "cuMemImportFromShareableHandle(fd)", __FILE__, __LINE__);
      break;
    }
    case CUMemHandleKind::kFabric: {
      CUmemFabricHandle fh;
      std::memcpy(&fh, data.fabric.data(), sizeof(fh));
      PPLX_CU_CHECK(cu.cuMemImportFromShareableHandle(&h, &fh, CU_MEM_HANDLE_TYPE_FABRIC));
      break;
    }
    default:
      throw Error(ErrorKind::kInvalidArgument, "cannot import a Local handle");
  }
  return h;
}
}  // namespace

CUMemImportHandle::CUMemImportHandle(const CUMemExportData& data, int device) {
  PPLX_REQUIRE(!data.multicast, "this export handle names a multicast object");
  cu_ensure_context(device);
  device_ = device;
  size_ = data.size;
  handle_ = import_generic(data);
}

// ---------------------------------------------------------------------------
// multicast objects (NVLS)
// ---------------------------------------------------------------------------

bool CUMulticastHandle::supported(int device) {
  if (!CuDriver::available()) return false;
  const CuDriver& cu = CuDriver::get();
  if (cu.cuMulticastCreate == nullptr) return false;
  CUdevice dev;
  if (cu.cuDeviceGet(&dev, device) != CUDA_SUCCESS) return false;
  int v = 0;
  if (cu.cuDeviceGetAttribute(&v, CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED, dev) != CUDA_SUCCESS) {
    return false;
  }
  return v != 0;
}

CUMulticastHandle::CUMulticastHandle(int num_devices, size_t size, CUMemHandleKind kind)
    : kind_(kind), num_devices_(num_devices) {
  const CuDriver& cu = CuDriver::get();
  PPLX_REQUIRE(cu.cuMulticastCreate != nullptr, "this CUDA driver has no multicast objects");
  PPLX_REQUIRE(num_devices > 0 && size > 0, "CUMulticastHandle: bad arguments");
  CUmulticastObjectProp prop{};
  prop.numDevices = static_cast<unsigned int>(num_devices);
  prop.handleTypes = cu_handle_type(kind);
  prop.size = size;
  size_t gran = 0;
  PPLX_CU_CHECK(cu.cuMulticastGetGranularity(&gran, &prop, CU_MULTICAST_GRANULARITY_RECOMMENDED));
  size_ = (size + gran - 1) / gran * gran;
  prop.size = size_;
  PPLX_CU_CHECK(cu.cuMulticastCreate(&handle_, &prop));
  int cur = 0;
  if (cudaGetDevice(&cur) == cudaSuccess) device_ = cur;
}

CUMulticastHandle::CUMulticastHandle(const CUMemExportData& data, int device)
    : kind_(data.kind), num_devices_(data.num_devices) {
  PPLX_REQUIRE(data.multicast, "this export handle does not name a multicast object");
  cu_ensure_context(device);
  device_ = device;
  size_ = data.size;
  handle_ = import_generic(data);
}

void CUMulticastHandle::unbind() {
  if (bound_bytes_ == 0) return;
  const CuDriver& cu = CuDriver::get();
  CUdevice dev;
  PPLX_CU_CHECK(cu.cuDeviceGet(&dev, bound_device_));
  PPLX_CU_CHECK(cu.cuMulticastUnbind(handle_, dev, 0, bound_bytes_));
  bound_bytes_ = 0;
}

CUMulticastHandle::~CUMulticastHandle() {
  if (bound_bytes_ != 0) {
    try {
      unbind();
    } catch (const std::exception&) {
      // nothing more can be done in a destructor
    }
  }
  if (exported_fd_ >= 0) {
    fd_server_unregister(exported_fd_);
    close(exported_fd_);
  }
}

void CUMulticastHandle::add_device(int device) {
  const CuDriver& cu = CuDriver::get();
  CUdevice dev;
  PPLX_CU_CHECK(cu.cuDeviceGet(&dev, device));
  PPLX_CU_CHECK(cu.cuMulticastAddDevice(handle_, dev));
  device_ = device;
}

void CUMulticastHandle::bind_mem(const CUAllocHandleBase& alloc) {
  const CuDriver& cu = CuDriver::get();
  PPLX_REQUIRE(alloc.size() <= size_, "bind_mem: the allocation is larger than the multicast object");
  PPLX_REQUIRE(bound_bytes_ == 0, "bind_mem: this process has already bound memory to the object");
  PPLX_CU_CHECK(cu.cuMulticastBindMem(handle_, 0, alloc.raw(), 0, alloc.size(), 0));
  bound_bytes_ = alloc.size();
  bound_device_ = alloc.device() >= 0 ? alloc.device() : device_;
}

CUMemExportData CUMulticastHandle::export_handle() {
  const CuDriver& cu = CuDriver::get();
  CUMemExportData d;
  d.kind = kind_;
  d.size = size_;
  d.device = device_;
  d.pid = getpid();
  d.multicast = true;
  d.num_devices = num_devices_;
  switch (kind_) {
    case CUMemHandleKind::kFileDescriptor: {
      if (exported_fd_ < 0) {
        int fd = -1;
        PPLX_CU_CHECK(cu.cuMemExportToShareableHandle(
            &fd, handle_, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0));
        exported_fd_ = fd;
        fd_server_register(fd);
      }
      d.fd = exported_fd_;
      d.socket_name = fd_server_name();
      break;
    }
    case CUMemHandleKind::kFabric: {
      CUmemFabricHandle fh;
      PPLX_CU_CHECK(cu.cuMemExportToShareableHandle(&fh, handle_, CU_MEM_HANDLE_TYPE_FABRIC, 0));
      std::memcpy(d.fabric.data(), &fh, sizeof(fh));
      break;
    }
    default:
      throw Error(ErrorKind::kInvalidArgument, "a Local multicast object cannot be exported");
  }
  return d;
}

}  // namespace pplx
