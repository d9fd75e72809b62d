#include "topo.h"

#include <cuda_runtime.h>
#include <dirent.h>

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
  };
  std::vector<Raw> raws;
  std::map<int, std::vector<int>> devices_of_numa;
  for (int dev = 0; dev < count; ++dev) {
    char bus[32] = {0};
    Raw raw{dev, 0, {}};
    if (cudaDeviceGetPCIBusId(bus, sizeof(bus), dev) == cudaSuccess) {
      std::string id(bus);
      std::transform(id.begin(), id.end(), id.begin(), ::tolower);
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
  for (const Raw& raw : raws) {
    TopologyGroup g;
    g.cuda_device = raw.device;
    g.numa = raw.numa;
    const std::vector<int>& siblings = devices_of_numa[raw.numa];
    const size_t index = static_cast<size_t>(std::find(siblings.begin(), siblings.end(), raw.device) - siblings.begin());
    g.cpus = split_evenly(raw.local_cpus, siblings.size(), index);
    if (g.cpus.size() < 3) g.cpus = raw.local_cpus;  // never starve a GPU of worker cores
    g.domains.push_back(DomainInfo{"nvl0:cuda" + std::to_string(raw.device), 7200ull * 1000 * 1000 * 1000, "local"});
    groups.push_back(std::move(g));
  }
  return groups;
}

}  // namespace

const std::vector<TopologyGroup>& detect_topology() {
  static std::vector<TopologyGroup> cached;
  static std::once_flag once;
  std::call_once(once, [] { cached = detect(); });
  return cached;
}

}  // namespace pplx::fabric
