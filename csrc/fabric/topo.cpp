#include "topo.h"

#include <cuda_runtime.h>
#include <dirent.h>
#include <dlfcn.h>

#include <algorithm>
#include <fstream>
#include <map>
#include <mutex>
#include <set>
#include <sstream>

#include "../core/thread_util.h"

namespace pplx::fabric {

std::vector<int> parse_cpu_list(const std::string& text) {
  std::vector<int> out;
  std::stringstream ss(text);
  std::string item;
  while (std::getline(ss, item, ',')) {
    while (!item.empty() && (item.back() == '\n' || item.back() == ' ')) item.pop_back();
    if (item.empty()) continue;
    const size_t dash = item.find('-');
    try {
      if (dash == std::string::npos) {
        out.push_back(std::stoi(item));
      } else {
        const int lo = std::stoi(item.substr(0, dash)), hi = std::stoi(item.substr(dash + 1));
        for (int c = lo; c <= hi; ++c) out.push_back(c);
      }
    } catch (...) {
      // ignore malformed pieces
    }
  }
  return out;
}

std::vector<int> split_evenly(const std::vector<int>& cpus, size_t parts, size_t index) {
  if (parts == 0 || index >= parts) return {};
  const size_t base = cpus.size() / parts, extra = cpus.size() % parts;
  const size_t begin = index * base + std::min(index, extra);
  const size_t len = base + (index < extra ? 1 : 0);
  return std::vector<int>(cpus.begin() + static_cast<long>(begin), cpus.begin() + static_cast<long>(begin + len));
}

namespace {

std::string read_file(const std::string& path) {
  std::ifstream in(path);
  std::stringstream ss;
  ss << in.rdbuf();
  return ss.str();
}

// Keeps one logical CPU per physical core (the lowest sibling).
std::vector<int> physical_cores(const std::vector<int>& cpus) {
  std::vector<int> out;
  std::set<int> seen;
  for (int c : cpus) {
    const std::string sib = read_file("/sys/devices/system/cpu/cpu" + std::to_string(c) + "/topology/thread_siblings_list");
    const std::vector<int> siblings = parse_cpu_list(sib);
    const int leader = siblings.empty() ? c : *std::min_element(siblings.begin(), siblings.end());
    if (seen.insert(leader).second) out.push_back(leader);
  }
  return out;
}

std::vector<TopologyGroup> detect() {
  std::vector<TopologyGroup> groups;
  const std::vector<int> allowed = current_affinity();
  const std::set<int> allowed_set(allowed.begin(), allowed.end());
  int count = 0;
  if (cudaGetDeviceCount(&count) != cudaSuccess) {
    cudaGetLastError();
    count = 0;
  }
  if (count == 0) {
    TopologyGroup g;
    g.cuda_device = -1;
    g.domains.push_back(DomainInfo{"host0", 100ull * 1000 * 1000 * 1000, "local"});
    g.cpus = allowed;
    groups.push_back(std::move(g));
    return groups;
  }
  struct Raw {
    int device, numa;
    std::vector<int> local_cpus;
    std::string pci_address;
  };
  std::vector<Raw> raws;
  std::map<int, std::vector<int>> devices_of_numa;
  for (int dev = 0; dev < count; ++dev) {
    char bus[32] = {0};
    Raw raw{dev, 0, {}};
    if (cudaDeviceGetPCIBusId(bus, sizeof(bus), dev) == cudaSuccess) {
      std::string id(bus);
      std::transform(id.begin(), id.end(), id.begin(), ::tolower);
      raw.pci_address = id;
      const std::string base = "/sys/bus/pci/devices/" + id;
      const std::string numa = read_file(base + "/numa_node");
      try {
        raw.numa = std::max(0, std::stoi(numa));
      } catch (...) {
        raw.numa = 0;
      }
      raw.local_cpus = parse_cpu_list(read_file(base + "/local_cpulist"));
    } else {
      cudaGetLastError();
    }
    if (raw.local_cpus.empty()) raw.local_cpus = allowed;
    std::vector<int> usable;
    for (int c : raw.local_cpus) {
      if (allowed_set.empty() || allowed_set.count(c)) usable.push_back(c);
    }
    if (usable.empty()) usable = allowed;
    raw.local_cpus = physical_cores(usable);
    if (raw.local_cpus.size() < 3) raw.local_cpus = usable;  // few cores: hyper-threads are better than nothing
    devices_of_numa[raw.numa].push_back(dev);
    raws.push_back(std::move(raw));
  }
  std::vector<std::string> gpu_addresses;
  for (const Raw& raw : raws) gpu_addresses.push_back(raw.pci_address);
  const std::vector<PciGpuPlacement> placement = place_gpus(scan_pci("/sys"), gpu_addresses);
  for (size_t ri = 0; ri < raws.size(); ++ri) {
    const Raw& raw = raws[ri];
    TopologyGroup g;
    g.cuda_device = raw.device;
    g.numa = raw.numa;
    g.pci_address = raw.pci_address;
    g.pci_switch = placement[ri].pci_switch;
    for (const PciNic& nic : placement[ri].nics) {
      const std::string rate = read_file("/sys/class/infiniband/" + nic.name + "/ports/1/rate");  // "400 Gb/sec (4X NDR)"
      uint64_t bits = 0;
      try {
        bits = static_cast<uint64_t>(std::stod(rate) * 1e9);
      } catch (...) {
        bits = 0;
      }
      g.nics.push_back(DomainInfo{nic.name, bits, "unavailable"});
    }
    const std::vector<int>& siblings = devices_of_numa[raw.numa];
    const size_t index = static_cast<size_t>(std::find(siblings.begin(), siblings.end(), raw.device) - siblings.begin());
    g.cpus = split_evenly(raw.local_cpus, siblings.size(), index);
    if (g.cpus.size() < 3) g.cpus = raw.local_cpus;  // never starve a GPU of worker cores
    uint64_t nvlink = nvlink_bits_per_second(raw.device);
    if (nvlink == 0) nvlink = 7200ull * 1000 * 1000 * 1000;  // NVLink 5: 18 links x 50 GB/s per direction
    g.domains.push_back(DomainInfo{"nvl0:cuda" + std::to_string(raw.device), nvlink, "local"});
    groups.push_back(std::move(g));
  }
  return groups;
}

}  // namespace

uint64_t nvlink_bits_per_second(int cuda_device) {
  // NVML is asked through dlopen so that nothing links against the driver's libraries.
  struct FieldValue {  // nvmlFieldValue_t
    uint32_t field_id, scope_id;
    int64_t timestamp, latency_usec;
    uint32_t value_type, nvml_return;
    union {
      double d;
      uint32_t ui;
      unsigned long ul;
      unsigned long long ull;
      long long sll;
    } value;
  };
  using InitFn = int (*)();
  using HandleFn = int (*)(const char*, void**);
  using FieldsFn = int (*)(void*, int, FieldValue*);
  static void* lib = dlopen("libnvidia-ml.so.1", RTLD_NOW | RTLD_LOCAL);
  if (lib == nullptr) return 0;
  static const auto init = reinterpret_cast<InitFn>(dlsym(lib, "nvmlInit_v2"));
  static const auto by_bus = reinterpret_cast<HandleFn>(dlsym(lib, "nvmlDeviceGetHandleByPciBusId_v2"));
  static const auto fields = reinterpret_cast<FieldsFn>(dlsym(lib, "nvmlDeviceGetFieldValues"));
  if (init == nullptr || by_bus == nullptr || fields == nullptr || init() != 0) return 0;
  char bus[32] = {0};
  if (cudaDeviceGetPCIBusId(bus, sizeof(bus), cuda_device) != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  void* handle = nullptr;
  if (by_bus(bus, &handle) != 0) return 0;
  FieldValue v[2] = {};
  v[0].field_id = 90;  // NVML_FI_DEV_NVLINK_SPEED_MBPS_COMMON: MB/s per link and direction
  v[1].field_id = 91;  // NVML_FI_DEV_NVLINK_LINK_COUNT
  if (fields(handle, 2, v) != 0 || v[0].nvml_return != 0 || v[1].nvml_return != 0) return 0;
  const uint64_t mbps = v[0].value.ui, links = v[1].value.ui;
  return mbps * links * 8ull * 1000ull * 1000ull;
}

const std::vector<TopologyGroup>& detect_topology() {
  static std::vector<TopologyGroup> cached;
  static std::once_flag once;
  std::call_once(once, [] { cached = detect(); });
  return cached;
}

}  // namespace pplx::fabric
