#include "local_domain.h"

#include <sys/socket.h>
#include <sys/un.h>
#include <unistd.h>

#include <algorithm>
#include <atomic>
#include <cstring>
#include <random>

#include "../core/cu_driver.h"
#include "../core/error.h"
#define PPLX_LOG_TARGET "pplx_garden::fabric::local"
#include "../core/log.h"
#include "../cumem/cumem.h"
#include "peer_copy.h"

namespace pplx::fabric {

namespace {
// A one-sided write into host memory that another thread may be polling (a flag word after the
// data it announces): words are stored with release semantics, so that everything this thread
// copied before is visible to a reader that sees the word, also on weakly ordered CPUs; anything
// else is a plain copy.
void host_write(void* dst, const void* src, size_t n) {
  const uintptr_t d = reinterpret_cast<uintptr_t>(dst);
  if (n == 4 && d % 4 == 0) {
    uint32_t v;
    std::memcpy(&v, src, 4);
    __atomic_store_n(static_cast<uint32_t*>(dst), v, __ATOMIC_RELEASE);
  } else if (n == 8 && d % 8 == 0) {
    uint64_t v;
    std::memcpy(&v, src, 8);
    __atomic_store_n(static_cast<uint64_t*>(dst), v, __ATOMIC_RELEASE);
  } else {
    std::memcpy(dst, src, n);
  }
}
}  // namespace

namespace {

enum MsgType : uint32_t {
  kMsgSend = 1,
  kMsgImm = 2,
  kMsgMrQuery = 3,
  kMsgMrReply = 4,
  kMsgHostWrite = 5,
  kMsgHostWriteAck = 6,
};

struct WireHeader {
  uint32_t magic;
  uint32_t type;
  uint64_t a, b;
  uint32_t c;
  uint32_t len;
};
constexpr uint32_t kWireMagic = 0x4c424146;  // "FABL"
constexpr size_t kMaxDatagram = 60 * 1024;

struct MrInfoWire {
  uint64_t ptr, len;
  int32_t device;
  int32_t pid;
  int32_t has_ipc;
  uint32_t pad;
  uint64_t ipc_offset;
  cudaIpcMemHandle_t ipc;
  int32_t has_vmm;
  int32_t vmm_fd;
  uint64_t vmm_size;
  char vmm_socket[96];   // descriptor server of the owner, NUL terminated
};

std::mutex g_registry_mu;
std::map<DomainAddress, LocalDomain*>& registry() {
  static auto* r = new std::map<DomainAddress, LocalDomain*>();
  return *r;
}

socklen_t socket_addr(const DomainAddress& a, sockaddr_un* out) {
  std::memset(out, 0, sizeof(*out));
  out->sun_family = AF_UNIX;
  const std::string name = "pplx-fab-" + a.to_hex();
  const size_t n = std::min(name.size(), sizeof(out->sun_path) - 2);
  std::memcpy(out->sun_path + 1, name.data(), n);
  return static_cast<socklen_t>(offsetof(sockaddr_un, sun_path) + 1 + n);
}

DomainAddress address_from_socket(const sockaddr_un& addr, socklen_t len) {
  const size_t n = len - offsetof(sockaddr_un, sun_path) - 1;
  const std::string name(addr.sun_path + 1, n);
  const std::string prefix = "pplx-fab-";
  if (name.rfind(prefix, 0) != 0) return DomainAddress();
  try {
    return DomainAddress::from_hex(name.substr(prefix.size()));
  } catch (...) {
    return DomainAddress();
  }
}

int32_t address_pid(const DomainAddress& a) {
  int32_t pid = 0;
  if (a.bytes().size() >= 5) std::memcpy(&pid, a.bytes().data() + 1, 4);
  return pid;
}

}  // namespace

LocalDomain::LocalDomain(int device, int index) : device_(device) {
  // address = 'L' | pid | 8 random bytes | index
  std::random_device rd;
  std::string bytes = "L";
  const int32_t pid = getpid();
  bytes.append(reinterpret_cast<const char*>(&pid), 4);
  const uint64_t nonce = (static_cast<uint64_t>(rd()) << 32) | rd();
  bytes.append(reinterpret_cast<const char*>(&nonce), 8);
  const int32_t idx = index;
  bytes.append(reinterpret_cast<const char*>(&idx), 4);
  address_ = DomainAddress(bytes);
  info_.name = device >= 0 ? "nvl" + std::to_string(index) + ":cuda" + std::to_string(device)
                           : "host" + std::to_string(index);
  info_.provider = "local";
  // NVLink 5: 900 GB/s per direction per GPU; host-only domains are memcpy-bound
  info_.link_speed = device >= 0 ? 7200ull * 1000 * 1000 * 1000 : 100ull * 1000 * 1000 * 1000;

  sock_ = socket(AF_UNIX, SOCK_DGRAM | SOCK_NONBLOCK | SOCK_CLOEXEC, 0);
  if (sock_ < 0) throw Error::from_errno("socket(AF_UNIX, SOCK_DGRAM)");
  sockaddr_un sa;
  const socklen_t len = socket_addr(address_, &sa);
  if (bind(sock_, reinterpret_cast<sockaddr*>(&sa), len) != 0) {
    const int e = errno;
    close(sock_);
    throw Error::from_errno("bind(fabric control socket)", e);
  }
  int buf = 8 << 20;
  setsockopt(sock_, SOL_SOCKET, SO_RCVBUF, &buf, sizeof(buf));
  setsockopt(sock_, SOL_SOCKET, SO_SNDBUF, &buf, sizeof(buf));
  {
    std::lock_guard<std::mutex> lock(g_registry_mu);
    registry()[address_] = this;
  }
}

LocalDomain::~LocalDomain() {
  {
    std::lock_guard<std::mutex> lock(g_registry_mu);
    registry().erase(address_);
  }
  if (device_ >= 0 && stream_ != nullptr) {
    cudaSetDevice(device_);
    cudaStreamSynchronize(stream_);
    for (auto& f : in_flight_) {
      if (f.event) cudaEventDestroy(f.event);
    }
    for (auto& kv : remotes_) {
      if (kv.second.ipc_base != nullptr) cudaIpcCloseMemHandle(kv.second.ipc_base);
      if (kv.second.vmm_va != 0 && CuDriver::available()) {
        const CuDriver& cu = CuDriver::get();
        cu.cuMemUnmap(static_cast<CUdeviceptr>(kv.second.vmm_va), kv.second.vmm_size);
        cu.cuMemAddressFree(static_cast<CUdeviceptr>(kv.second.vmm_va), kv.second.vmm_size);
      }
    }
    if (scratch_) cudaFree(scratch_);
    if (error_flag_host_) cudaFreeHost(error_flag_host_);
    cudaStreamDestroy(stream_);
  }
  if (sock_ >= 0) close(sock_);
}

LocalDomain* LocalDomain::find_local(const DomainAddress& addr) {
  std::lock_guard<std::mutex> lock(g_registry_mu);
  auto it = registry().find(addr);
  return it == registry().end() ? nullptr : it->second;
}

void LocalDomain::ensure_stream() {
  if (device_ < 0 || stream_ != nullptr) return;
  PPLX_CUDA_CHECK(cudaSetDevice(device_));
  PPLX_CUDA_CHECK(cudaStreamCreateWithFlags(&stream_, cudaStreamNonBlocking));
  PPLX_CUDA_CHECK(cudaHostAlloc(reinterpret_cast<void**>(&error_flag_host_), 64, cudaHostAllocMapped));
  std::memset(error_flag_host_, 0, 64);
  PPLX_CUDA_CHECK(cudaHostGetDevicePointer(reinterpret_cast<void**>(&error_flag_dev_), error_flag_host_, 0));
  // Everything a later write could otherwise allocate or load lazily is set up here, at
  // registration time: a write may be submitted while a kernel that waits for it fills the GPU,
  // and cudaMalloc or a first kernel launch can then block behind that very kernel.
  device_scratch(1u << 17);
  PPLX_CUDA_CHECK(warm_up_paged_copy(stream_));
}

uint32_t* LocalDomain::device_scratch(size_t words) {
  if (words > scratch_words_) {
    if (scratch_ != nullptr) {
      PPLX_CUDA_CHECK(cudaStreamSynchronize(stream_));
      PPLX_CUDA_CHECK(cudaFree(scratch_));
    }
    size_t cap = 4096;
    while (cap < words) cap <<= 1;
    PPLX_CUDA_CHECK(cudaMalloc(reinterpret_cast<void**>(&scratch_), cap * sizeof(uint32_t)));
    scratch_words_ = cap;
  }
  return scratch_;
}

// ---------------------------------------------------------------------------
// memory regions
// ---------------------------------------------------------------------------

MemoryRegionRemoteKey LocalDomain::register_mr(uint64_t ptr, uint64_t len, int device) {
  std::lock_guard<std::mutex> lock(regions_mu_);
  auto it = regions_.find(ptr);
  if (it != regions_.end()) return it->second.rkey;
  Region r;
  r.ptr = ptr;
  r.len = len;
  r.device = device;
  r.rkey = next_rkey_++;
  if (device >= 0 && device_ >= 0) ensure_stream();
  if (device >= 0) {
    // A CUDA IPC handle names a whole allocation: find its base so that peers in other
    // processes can map it and add the offset of this region.
    PPLX_CUDA_CHECK(cudaSetDevice(device));
    const CuDriver& cu = CuDriver::get();
    CUdeviceptr base = 0;
    size_t size = 0;
    if (cu.cuMemGetAddressRange(&base, &size, static_cast<CUdeviceptr>(ptr)) == CUDA_SUCCESS) {
      cudaIpcMemHandle_t h;
      if (cudaIpcGetMemHandle(&h, reinterpret_cast<void*>(base)) == cudaSuccess) {
        r.has_ipc = true;
        r.ipc = h;
        r.ipc_offset = ptr - static_cast<uint64_t>(base);
      } else {
        cudaGetLastError();
        // not cudaMalloc memory; a virtual-memory allocation can be shared as a file descriptor
        CUmemGenericAllocationHandle handle;
        if (cu.cuMemRetainAllocationHandle != nullptr &&
            cu.cuMemRetainAllocationHandle(&handle, reinterpret_cast<void*>(ptr)) == CUDA_SUCCESS) {
          int fd = -1;
          if (cu.cuMemExportToShareableHandle(&fd, handle, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0) ==
              CUDA_SUCCESS) {
            r.vmm_fd = fd;
            r.vmm_size = size;
            r.ipc_offset = ptr - static_cast<uint64_t>(base);
            fd_server_register(fd);
          }
          cu.cuMemRelease(handle);   // the retain above took a reference
        }
      }
    }
  }
  by_rkey_[r.rkey] = ptr;
  regions_[ptr] = r;
  return r.rkey;
}

void LocalDomain::unregister_mr(uint64_t ptr) {
  std::lock_guard<std::mutex> lock(regions_mu_);
  auto it = regions_.find(ptr);
  if (it == regions_.end()) return;
  if (it->second.vmm_fd >= 0) {
    fd_server_unregister(it->second.vmm_fd);
    close(it->second.vmm_fd);
  }
  by_rkey_.erase(it->second.rkey);
  regions_.erase(it);
}

std::string LocalDomain::region_info(const Region& r) const {
  MrInfoWire w{};
  w.ptr = r.ptr;
  w.len = r.len;
  w.device = r.device;
  w.pid = getpid();
  w.has_ipc = r.has_ipc ? 1 : 0;
  w.ipc_offset = r.ipc_offset;
  w.ipc = r.ipc;
  if (r.vmm_fd >= 0) {
    w.has_vmm = 1;
    w.vmm_fd = r.vmm_fd;
    w.vmm_size = r.vmm_size;
    const std::string name = fd_server_name();
    std::strncpy(w.vmm_socket, name.c_str(), sizeof(w.vmm_socket) - 1);
  }
  return std::string(reinterpret_cast<const char*>(&w), sizeof(w));
}

// ---------------------------------------------------------------------------
// messaging
// ---------------------------------------------------------------------------

void LocalDomain::deliver(const DomainAddress& dst, Message msg) {
  msg.from = address_;
  if (LocalDomain* peer = find_local(dst)) {
    std::lock_guard<std::mutex> lock(peer->inbox_mu_);
    peer->inbox_.push_back(std::move(msg));
    return;
  }
  if (msg.payload.size() > kMaxDatagram) {
    throw Error(ErrorKind::kDomain, "control message too large for one datagram");
  }
  WireHeader h{kWireMagic, msg.type, msg.a, msg.b, msg.c, static_cast<uint32_t>(msg.payload.size())};
  iovec iov[2] = {{&h, sizeof(h)}, {const_cast<char*>(msg.payload.data()), msg.payload.size()}};
  sockaddr_un sa;
  const socklen_t len = socket_addr(dst, &sa);
  msghdr m{};
  m.msg_name = &sa;
  m.msg_namelen = len;
  m.msg_iov = iov;
  m.msg_iovlen = 2;
  for (int attempt = 0;; ++attempt) {
    if (sendmsg(sock_, &m, MSG_NOSIGNAL) >= 0) return;
    if ((errno == EAGAIN || errno == EWOULDBLOCK || errno == ENOBUFS) && attempt < 20000) {
      usleep(50);  // receiver's queue is full: back off, it drains from its worker thread
      continue;
    }
    throw Error::from_errno("sendmsg to domain " + dst.to_hex());
  }
}

void LocalDomain::drain_socket(std::vector<DomainCompletion>* out) {
  static thread_local std::vector<char> buf(sizeof(WireHeader) + kMaxDatagram + 64);
  for (int i = 0; i < 64; ++i) {
    sockaddr_un sa;
    socklen_t salen = sizeof(sa);
    const ssize_t n = recvfrom(sock_, buf.data(), buf.size(), MSG_DONTWAIT,
                               reinterpret_cast<sockaddr*>(&sa), &salen);
    if (n < 0) return;
    if (static_cast<size_t>(n) < sizeof(WireHeader)) continue;
    WireHeader h;
    std::memcpy(&h, buf.data(), sizeof(h));
    if (h.magic != kWireMagic || sizeof(WireHeader) + h.len != static_cast<size_t>(n)) continue;
    Message msg;
    msg.type = h.type;
    msg.a = h.a;
    msg.b = h.b;
    msg.c = h.c;
    msg.payload.assign(buf.data() + sizeof(h), h.len);
    msg.from = address_from_socket(sa, salen);
    handle(msg, out);
  }
}

void LocalDomain::handle(Message& msg, std::vector<DomainCompletion>* out) {
  switch (msg.type) {
    case kMsgSend: {
      if (recv_credits_.empty()) {
        unclaimed_.push_back(std::move(msg));
        return;
      }
      RecvCredit& credit = recv_credits_.front();
      DomainCompletion c;
      c.kind = DomainCompletion::Kind::kRecv;
      c.transfer_id = credit.id;
      c.data = std::move(msg.payload);
      if (c.data.size() > credit.len) {
        c.kind = DomainCompletion::Kind::kError;
        c.error = "received message longer than the posted buffer";
      }
      if (--credit.remaining == 0) recv_credits_.pop_front();
      out->push_back(std::move(c));
      return;
    }
    case kMsgImm: {
      DomainCompletion c;
      c.kind = DomainCompletion::Kind::kImm;
      c.imm = static_cast<uint32_t>(msg.a);
      c.imm_count = static_cast<uint32_t>(msg.b);
      out->push_back(std::move(c));
      return;
    }
    case kMsgMrQuery: {
      Message reply;
      reply.type = kMsgMrReply;
      reply.a = msg.a;
      {
        std::lock_guard<std::mutex> lock(regions_mu_);
        auto it = by_rkey_.find(msg.a);
        if (it != by_rkey_.end()) {
          reply.c = 1;
          reply.payload = region_info(regions_[it->second]);
        }
      }
      deliver(msg.from, std::move(reply));
      return;
    }
    case kMsgMrReply: {
      const auto key = std::make_pair(msg.from, static_cast<MemoryRegionRemoteKey>(msg.a));
      RemoteRegion& rr = remotes_[key];
      std::string failure;
      if (msg.c != 1 || msg.payload.size() != sizeof(MrInfoWire)) {
        failure = "the destination does not know this memory region key";
      } else {
        MrInfoWire w;
        std::memcpy(&w, msg.payload.data(), sizeof(w));
        rr.resolved = true;
        rr.same_process = false;
        rr.device = w.device;
        rr.owner_ptr = w.ptr;
        rr.len = w.len;
        if (w.device >= 0) {
          if (device_ < 0) {
            failure = "a host-only domain cannot write into another process's GPU memory";
          } else if (!w.has_ipc && w.has_vmm) {
            // a CUDA virtual-memory allocation: fetch its descriptor, import and map it here
            try {
              const CuDriver& cu = CuDriver::get();
              cudaSetDevice(device_);
              cu_ensure_context(device_);
              w.vmm_socket[sizeof(w.vmm_socket) - 1] = 0;
              const int fd = fd_fetch(w.pid, w.vmm_fd, w.vmm_socket);
              CUmemGenericAllocationHandle handle;
              const CUresult imported = cu.cuMemImportFromShareableHandle(
                  &handle, reinterpret_cast<void*>(static_cast<uintptr_t>(fd)), CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR);
              close(fd);
              PPLX_CU_CHECK(imported);
              CUdeviceptr va = 0;
              PPLX_CU_CHECK(cu.cuMemAddressReserve(&va, w.vmm_size, 0, 0, 0));
              CUresult mapped = cu.cuMemMap(va, w.vmm_size, 0, handle, 0);
              cu.cuMemRelease(handle);   // the mapping keeps the memory alive
              if (mapped == CUDA_SUCCESS) {
                CUmemAccessDesc access{};
                access.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
                access.location.id = device_;
                access.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
                mapped = cu.cuMemSetAccess(va, w.vmm_size, &access, 1);
                if (mapped != CUDA_SUCCESS) cu.cuMemUnmap(va, w.vmm_size);
              }
              if (mapped != CUDA_SUCCESS) {
                cu.cuMemAddressFree(va, w.vmm_size);
                PPLX_CU_CHECK(mapped);
              }
              rr.vmm_va = static_cast<uint64_t>(va);
              rr.vmm_size = w.vmm_size;
              rr.mapped = reinterpret_cast<uint8_t*>(va) + w.ipc_offset;
            } catch (const std::exception& e) {
              failure = std::string("importing the destination's virtual-memory allocation: ") + e.what();
            }
          } else if (!w.has_ipc) {
            failure = "the destination region cannot be shared between processes (no CUDA IPC handle)";
          } else {
            cudaSetDevice(device_);
            void* base = nullptr;
            const cudaError_t e = cudaIpcOpenMemHandle(&base, w.ipc, cudaIpcMemLazyEnablePeerAccess);
            if (e != cudaSuccess) {
              cudaGetLastError();
              failure = std::string("cudaIpcOpenMemHandle: ") + cudaGetErrorString(e);
            } else {
              rr.ipc_base = base;
              rr.mapped = static_cast<uint8_t*>(base) + w.ipc_offset;
            }
          }
        }
      }
      auto waiting = waiting_mr_.find(key);
      if (waiting == waiting_mr_.end()) return;
      std::vector<PendingWrite> ops = std::move(waiting->second);
      waiting_mr_.erase(waiting);
      for (PendingWrite& w : ops) {
        if (!failure.empty()) {
          DomainCompletion c;
          c.kind = DomainCompletion::Kind::kError;
          c.transfer_id = w.id;
          c.error = failure;
          out->push_back(std::move(c));
        } else {
          try {
            run_write(w, rr, out);
          } catch (const std::exception& e) {
            DomainCompletion c;
            c.kind = DomainCompletion::Kind::kError;
            c.transfer_id = w.id;
            c.error = e.what();
            out->push_back(std::move(c));
          }
        }
      }
      if (!failure.empty()) remotes_.erase(key);
      return;
    }
    case kMsgHostWrite: {
      std::unique_lock<std::mutex> lock(regions_mu_);
      auto it = by_rkey_.find(msg.a);
      const bool last = (msg.c & 1u) != 0;
      bool ok = false;
      if (it != by_rkey_.end()) {
        const Region& r = regions_[it->second];
        if (r.device < 0 && msg.b + msg.payload.size() <= r.len) {
          host_write(reinterpret_cast<void*>(r.ptr + msg.b), msg.payload.data(), msg.payload.size());
          ok = true;
        }
      }
      lock.unlock();
      if (last || !ok) {
        Message ack;
        ack.type = kMsgHostWriteAck;
        ack.b = ok ? 1 : 0;
        ack.c = msg.c;  // (ticket << 1 | last) of the sender
        deliver(msg.from, std::move(ack));
      }
      return;
    }
    case kMsgHostWriteAck: {
      // c carries (ticket << 1 | last); tickets are looked up in host_write_acks_
      const TransferId ticket = msg.c >> 1;
      auto it = host_write_acks_.find(ticket);
      if (it == host_write_acks_.end()) return;
      if (msg.b != 1) {
        DomainCompletion c;
        c.kind = DomainCompletion::Kind::kError;
        c.transfer_id = it->second;
        c.error = "the destination rejected a host write (bad key or out of bounds)";
        out->push_back(std::move(c));
      } else {
        DomainCompletion c;
        c.kind = DomainCompletion::Kind::kWriteDone;
        c.transfer_id = it->second;
        out->push_back(std::move(c));
      }
      host_write_acks_.erase(it);
      return;
    }
    default:
      PPLX_WARN("dropping control message of unknown type %u", msg.type);
  }
}

// ---------------------------------------------------------------------------
// writes
// ---------------------------------------------------------------------------

void LocalDomain::submit_send(TransferId transfer_id, const DomainAddress& dst, std::string data) {
  DomainCompletion c;
  c.transfer_id = transfer_id;
  try {
    Message m;
    m.type = kMsgSend;
    m.payload = std::move(data);
    deliver(dst, std::move(m));
    c.kind = DomainCompletion::Kind::kSendDone;
  } catch (const std::exception& e) {
    c.kind = DomainCompletion::Kind::kError;
    c.error = e.what();
  }
  ready_.push_back(std::move(c));
}

void LocalDomain::post_recvs(TransferId transfer_id, size_t count, size_t len) {
  if (count == 0) return;
  recv_credits_.push_back(RecvCredit{transfer_id, count, len});
}

void LocalDomain::submit_write(TransferId transfer_id, const DomainAddress& dst, WriteOp op) {
  ++writes_submitted_;
  if (fail_write_at_ != 0 && writes_submitted_ == fail_write_at_) {
    DomainCompletion c;
    c.kind = DomainCompletion::Kind::kError;
    c.transfer_id = transfer_id;
    c.error = "injected write failure";
    ready_.push_back(std::move(c));
    return;
  }
  PendingWrite w{transfer_id, dst, std::move(op)};
  std::vector<DomainCompletion> out;
  try {
    start_write(std::move(w), &out);
  } catch (const std::exception& e) {
    DomainCompletion c;
    c.kind = DomainCompletion::Kind::kError;
    c.transfer_id = transfer_id;
    c.error = e.what();
    out.push_back(std::move(c));
  }
  for (auto& c : out) ready_.push_back(std::move(c));
}

LocalDomain::RemoteRegion& LocalDomain::remote(const DomainAddress& dst, MemoryRegionRemoteKey rkey) {
  return remotes_[std::make_pair(dst, rkey)];
}

void LocalDomain::start_write(PendingWrite w, std::vector<DomainCompletion>* out) {
  if (w.op.kind == WriteOp::Kind::kImm) {
    Message m;
    m.type = kMsgImm;
    m.a = w.op.imm.imm_data;
    m.b = 1;
    deliver(w.dst, std::move(m));
    DomainCompletion c;
    c.kind = DomainCompletion::Kind::kWriteDone;
    c.transfer_id = w.id;
    out->push_back(std::move(c));
    return;
  }
  const MemoryRegionRemoteKey rkey =
      w.op.kind == WriteOp::Kind::kSingle ? w.op.single.dst_rkey : w.op.paged.dst_rkey;
  const auto key = std::make_pair(w.dst, rkey);
  RemoteRegion& rr = remotes_[key];
  if (!rr.resolved) {
    if (LocalDomain* peer = find_local(w.dst)) {
      // same process: look the region up directly
      std::lock_guard<std::mutex> lock(peer->regions_mu_);
      auto it = peer->by_rkey_.find(rkey);
      if (it == peer->by_rkey_.end()) {
        remotes_.erase(key);
        throw Error(ErrorKind::kDomain, "the destination does not know this memory region key");
      }
      const Region& r = peer->regions_[it->second];
      rr.resolved = true;
      rr.same_process = true;
      rr.device = r.device;
      rr.owner_ptr = r.ptr;
      rr.len = r.len;
      rr.mapped = reinterpret_cast<uint8_t*>(r.ptr);
      if (r.device >= 0 && device_ >= 0 && r.device != device_) {
        cudaSetDevice(device_);
        const cudaError_t e = cudaDeviceEnablePeerAccess(r.device, 0);
        if (e != cudaSuccess && e != cudaErrorPeerAccessAlreadyEnabled) {
          remotes_.erase(key);
          throw Error(ErrorKind::kCudaRuntime, std::string("cudaDeviceEnablePeerAccess: ") + cudaGetErrorString(e));
        }
        cudaGetLastError();
      }
    } else {
      auto& queue = waiting_mr_[key];
      const bool first = queue.empty();
      queue.push_back(std::move(w));
      if (first) {
        Message q;
        q.type = kMsgMrQuery;
        q.a = rkey;
        deliver(key.first, std::move(q));
      }
      return;
    }
  }
  run_write(w, rr, out);
}

void LocalDomain::run_write(const PendingWrite& w, RemoteRegion& rr, std::vector<DomainCompletion>* out) {
  // Normalise both kinds of write into "pages".
  uint64_t src_base, length, src_stride, src_offset, dst_stride, dst_offset;
  const std::vector<uint32_t>* src_pages = nullptr;
  const std::vector<uint32_t>* dst_pages = nullptr;
  size_t page_begin = 0, page_end = 1;
  std::optional<uint32_t> imm;
  if (w.op.kind == WriteOp::Kind::kSingle) {
    const SingleWriteOp& s = w.op.single;
    src_base = s.src_ptr;
    length = s.length;
    src_stride = dst_stride = 0;
    src_offset = s.src_offset;
    dst_offset = s.dst_offset;
    imm = s.imm_data;
  } else {
    const PagedWriteOp& p = w.op.paged;
    src_base = p.src_ptr;
    length = p.length;
    src_stride = p.src_stride;
    dst_stride = p.dst_stride;
    src_offset = p.src_offset;
    dst_offset = p.dst_offset;
    src_pages = p.src_page_indices.get();
    dst_pages = p.dst_page_indices.get();
    page_begin = p.page_begin;
    page_end = p.page_end;
    imm = p.imm_data;
  }
  const size_t num_pages = page_end - page_begin;
  auto src_page = [&](size_t i) { return src_pages ? (*src_pages)[page_begin + i] : 0u; };
  auto dst_page = [&](size_t i) { return dst_pages ? (*dst_pages)[page_begin + i] : 0u; };
  // Bounds of both sides, checked on the host before anything is enqueued: an index, stride
  // or offset that leaves a registered region would otherwise become an out-of-range device
  // access (the RDMA providers of the reference get this check from the lkey / rkey).
  auto span_end = [](uint64_t page, uint64_t stride, uint64_t offset, uint64_t len, uint64_t* end) {
    unsigned __int128 e = static_cast<unsigned __int128>(page) * stride;
    e += offset;
    e += len;
    if (e > UINT64_MAX) return false;
    *end = static_cast<uint64_t>(e);
    return true;
  };
  for (size_t i = 0; i < num_pages && length > 0; ++i) {
    uint64_t end = 0;
    if (!span_end(dst_page(i), dst_stride, dst_offset, length, &end) || end > rr.len) {
      throw Error(ErrorKind::kDomain, "write past the end of the destination region");
    }
  }

  // source region: its device, and its extent
  int src_device = -1;
  {
    uint64_t region_ptr = 0, region_len = 0;
    bool found = false;
    {
      std::lock_guard<std::mutex> lock(regions_mu_);
      auto it = regions_.upper_bound(src_base);
      if (it != regions_.begin()) {
        --it;
        if (src_base < it->second.ptr + it->second.len) {
          src_device = it->second.device;
          region_ptr = it->second.ptr;
          region_len = it->second.len;
          found = true;
        }
      }
    }
    if (!found && length > 0 && num_pages > 0) {
      throw Error(ErrorKind::kDomain, "the source of a write is not inside a registered region");
    }
    const uint64_t base_off = src_base - region_ptr;
    for (size_t i = 0; i < num_pages && length > 0; ++i) {
      uint64_t end = 0;
      if (!span_end(src_page(i), src_stride, src_offset, length, &end) || end > region_len ||
          base_off > region_len - end) {
        throw Error(ErrorKind::kDomain, "read past the end of the source region");
      }
    }
  }

  auto finish_now = [&]() {
    if (imm.has_value()) {
      Message m;
      m.type = kMsgImm;
      m.a = *imm;
      m.b = std::max<size_t>(num_pages, 1);
      deliver(w.dst, std::move(m));
    }
    DomainCompletion c;
    c.kind = DomainCompletion::Kind::kWriteDone;
    c.transfer_id = w.id;
    out->push_back(std::move(c));
  };

  if (length == 0 || num_pages == 0) {
    finish_now();
    return;
  }

  const bool dst_dev = rr.device >= 0;
  const bool src_dev = src_device >= 0;

  if (!dst_dev && !src_dev) {
    if (rr.same_process) {
      for (size_t i = 0; i < num_pages; ++i) {
        host_write(rr.mapped + dst_page(i) * dst_stride + dst_offset,
                   reinterpret_cast<const void*>(src_base + src_page(i) * src_stride + src_offset), length);
      }
      finish_now();
      return;
    }
    // host -> host across processes: ship the bytes over the control socket
    static std::atomic<uint32_t> next_ticket{1};
    const uint32_t ticket = next_ticket.fetch_add(1) & 0x7fffffffu;
    const MemoryRegionRemoteKey rkey =
        w.op.kind == WriteOp::Kind::kSingle ? w.op.single.dst_rkey : w.op.paged.dst_rkey;
    host_write_acks_[ticket] = w.id;
    for (size_t i = 0; i < num_pages; ++i) {
      const char* src = reinterpret_cast<const char*>(src_base + src_page(i) * src_stride + src_offset);
      const uint64_t dst_off = dst_page(i) * dst_stride + dst_offset;
      for (uint64_t done = 0; done < length; done += kMaxDatagram) {
        const uint64_t n = std::min<uint64_t>(kMaxDatagram, length - done);
        Message m;
        m.type = kMsgHostWrite;
        m.a = rkey;
        m.b = dst_off + done;
        const bool last = (i + 1 == num_pages) && (done + n == length);
        m.c = (ticket << 1) | (last ? 1u : 0u);
        m.payload.assign(src + done, n);
        deliver(w.dst, std::move(m));
      }
    }
    // unix datagrams between two sockets are delivered in order: the immediate follows the data
    if (imm.has_value()) {
      Message m;
      m.type = kMsgImm;
      m.a = *imm;
      m.b = std::max<size_t>(num_pages, 1);
      deliver(w.dst, std::move(m));
    }
    return;  // completion arrives with the acknowledgement
  }

  if (device_ < 0) throw Error(ErrorKind::kDomain, "a host-only domain cannot move GPU memory");
  if (dst_dev && rr.mapped == nullptr) throw Error(ErrorKind::kDomain, "destination GPU region is not mapped");
  if (!dst_dev && !rr.same_process) {
    throw Error(ErrorKind::kDomain, "GPU to remote-process host memory is not supported by the local provider");
  }
  ensure_stream();
  PPLX_CUDA_CHECK(cudaSetDevice(device_));

  if (dst_dev && src_dev && num_pages == 1 && src_pages == nullptr) {
    // One contiguous range: the copy engines move it, no SM is needed. That matters to callers
    // whose own kernels fill the GPU while they wait for this very copy (the all-to-all proxy).
    PPLX_CUDA_CHECK(cudaMemcpyAsync(rr.mapped + dst_offset, reinterpret_cast<const void*>(src_base + src_offset),
                                    length, cudaMemcpyDeviceToDevice, stream_));
  } else if (dst_dev && src_dev) {
    PagedCopyArgs a{};
    a.src_base = reinterpret_cast<const uint8_t*>(src_base);
    a.dst_base = rr.mapped;
    a.src_stride = src_stride;
    a.dst_stride = dst_stride;
    a.src_offset = src_offset;
    a.dst_offset = dst_offset;
    a.length = length;
    a.num_pages = static_cast<uint32_t>(num_pages);
    a.error_flag = error_flag_dev_;
    if (src_pages != nullptr) {
      uint32_t* scratch = device_scratch(2 * num_pages);
      PPLX_CUDA_CHECK(cudaMemcpyAsync(scratch, src_pages->data() + page_begin, num_pages * sizeof(uint32_t),
                                      cudaMemcpyHostToDevice, stream_));
      PPLX_CUDA_CHECK(cudaMemcpyAsync(scratch + num_pages, dst_pages->data() + page_begin,
                                      num_pages * sizeof(uint32_t), cudaMemcpyHostToDevice, stream_));
      a.src_pages = scratch;
      a.dst_pages = scratch + num_pages;
    }
    // CTAs of the bulk-copy kernel: PPLX_COPY_CTAS overrides the default (a fraction of the SMs)
    static const int copy_ctas = [] {
      const char* env = std::getenv("PPLX_COPY_CTAS");
      return env != nullptr ? std::atoi(env) : 0;
    }();
    PPLX_CUDA_CHECK(launch_paged_copy(a, copy_ctas, stream_));
  } else {
    // one side is host memory of this process: let the copy engine move each page
    for (size_t i = 0; i < num_pages; ++i) {
      void* dst = rr.mapped + dst_page(i) * dst_stride + dst_offset;
      const void* src = reinterpret_cast<const void*>(src_base + src_page(i) * src_stride + src_offset);
      PPLX_CUDA_CHECK(cudaMemcpyAsync(dst, src, length, cudaMemcpyDefault, stream_));
    }
  }
  InFlight f;
  f.id = w.id;
  f.dst = w.dst;
  f.has_imm = imm.has_value();
  f.imm = imm.value_or(0);
  f.imm_count = static_cast<uint32_t>(std::max<size_t>(num_pages, 1));
  f.error_flag = error_flag_host_;
  PPLX_CUDA_CHECK(cudaEventCreateWithFlags(&f.event, cudaEventDisableTiming));
  PPLX_CUDA_CHECK(cudaEventRecord(f.event, stream_));
  in_flight_.push_back(std::move(f));
}

// ---------------------------------------------------------------------------
// progress
// ---------------------------------------------------------------------------

void LocalDomain::poll_progress(std::vector<DomainCompletion>* out) {
  while (!ready_.empty()) {
    out->push_back(std::move(ready_.front()));
    ready_.pop_front();
  }
  // messages that waited for a receive to be posted
  while (!unclaimed_.empty() && !recv_credits_.empty()) {
    Message m = std::move(unclaimed_.front());
    unclaimed_.pop_front();
    handle(m, out);
  }
  {
    std::deque<Message> local;
    {
      std::lock_guard<std::mutex> lock(inbox_mu_);
      local.swap(inbox_);
    }
    for (Message& m : local) handle(m, out);
  }
  drain_socket(out);
  // copies complete in stream order
  while (!in_flight_.empty()) {
    InFlight& f = in_flight_.front();
    const cudaError_t e = cudaEventQuery(f.event);
    if (e == cudaErrorNotReady) {
      cudaGetLastError();
      if (++stuck_polls_ == 2000000) {
        PPLX_WARN("a copy of transfer %llu on %s has not completed after %llu polls (%zu in flight)",
                  static_cast<unsigned long long>(f.id), info_.name.c_str(),
                  static_cast<unsigned long long>(stuck_polls_), in_flight_.size());
      }
      break;
    }
    stuck_polls_ = 0;
    DomainCompletion c;
    c.transfer_id = f.id;
    if (e != cudaSuccess) {
      c.kind = DomainCompletion::Kind::kError;
      c.error = std::string("copy failed: ") + cudaGetErrorString(e);
    } else if (f.error_flag != nullptr && *reinterpret_cast<volatile uint32_t*>(f.error_flag) != 0) {
      c.kind = DomainCompletion::Kind::kError;
      c.error = "the copy kernel gave up waiting for a bulk load";
      *reinterpret_cast<volatile uint32_t*>(f.error_flag) = 0;
    } else {
      c.kind = DomainCompletion::Kind::kWriteDone;
      if (f.has_imm) {
        try {
          Message m;
          m.type = kMsgImm;
          m.a = f.imm;
          m.b = f.imm_count;
          deliver(f.dst, std::move(m));
        } catch (const std::exception& ex) {
          c.kind = DomainCompletion::Kind::kError;
          c.error = ex.what();
        }
      }
    }
    cudaEventDestroy(f.event);
    in_flight_.pop_front();
    out->push_back(std::move(c));
  }
}

bool LocalDomain::busy() const {
  return !in_flight_.empty() || !ready_.empty() || !waiting_mr_.empty() || !host_write_acks_.empty();
}

}  // namespace pplx::fabric
