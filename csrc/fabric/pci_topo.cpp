#include "pci_topo.h"

#include <dirent.h>
#include <limits.h>
#include <stdlib.h>
#include <sys/stat.h>

#include <algorithm>
#include <fstream>
#include <sstream>

namespace pplx::fabric {

namespace {

std::string slurp(const std::string& path) {
  std::ifstream in(path);
  std::stringstream ss;
  ss << in.rdbuf();
  std::string s = ss.str();
  while (!s.empty() && (s.back() == '\n' || s.back() == ' ')) s.pop_back();
  return s;
}

uint32_t parse_hex(const std::string& s) {
  try {
    return static_cast<uint32_t>(std::stoul(s, nullptr, 16));
  } catch (...) {
    return 0;
  }
}

// "0000:1b:00.0": four hex digits, colon, two, colon, two, dot, one.
bool looks_like_pci_address(const std::string& s) {
  if (s.size() != 12) return false;
  for (size_t i = 0; i < s.size(); ++i) {
    const char c = s[i];
    if (i == 4 || i == 7) {
      if (c != ':') return false;
    } else if (i == 10) {
      if (c != '.') return false;
    } else if (!isxdigit(static_cast<unsigned char>(c))) {
      return false;
    }
  }
  return true;
}

std::vector<std::string> list_dir(const std::string& path) {
  std::vector<std::string> out;
  DIR* d = opendir(path.c_str());
  if (d == nullptr) return out;
  while (dirent* e = readdir(d)) {
    const std::string name = e->d_name;
    if (name != "." && name != "..") out.push_back(name);
  }
  closedir(d);
  std::sort(out.begin(), out.end());
  return out;
}

}  // namespace

std::vector<PciDevice> scan_pci(const std::string& sysfs_root) {
  std::vector<PciDevice> devices;
  const std::string dir = sysfs_root + "/bus/pci/devices";
  for (const std::string& name : list_dir(dir)) {
    if (!looks_like_pci_address(name)) continue;
    const std::string link = dir + "/" + name;
    char resolved[PATH_MAX];
    if (realpath(link.c_str(), resolved) == nullptr) continue;
    // .../pci0000:16/0000:16:01.0/0000:17:00.0/0000:18:08.0/0000:1b:00.0
    const std::string real(resolved);
    const size_t last = real.rfind('/');
    if (last == std::string::npos) continue;
    const size_t prev = real.rfind('/', last - 1);
    std::string parent = prev == std::string::npos ? "" : real.substr(prev + 1, last - prev - 1);
    if (!looks_like_pci_address(parent)) parent.clear();
    PciDevice d;
    d.address = name;
    d.parent = parent;
    d.vendor = parse_hex(slurp(real + "/vendor"));
    d.device = parse_hex(slurp(real + "/device"));
    d.pci_class = parse_hex(slurp(real + "/class"));
    try {
      d.numa = std::stoi(slurp(real + "/numa_node"));
    } catch (...) {
      d.numa = -1;
    }
    d.rdma_names = list_dir(real + "/infiniband");
    devices.push_back(std::move(d));
  }
  std::sort(devices.begin(), devices.end(),
            [](const PciDevice& a, const PciDevice& b) { return a.address < b.address; });

  std::map<std::string, int> children;
  std::map<std::string, std::string> parent_of;
  for (const PciDevice& d : devices) {
    parent_of[d.address] = d.parent;
    if (!d.parent.empty()) ++children[d.parent];
  }
  for (PciDevice& d : devices) {
    // climb while the bridge above has this subtree as its only child
    std::string at = d.parent;
    if (at.empty()) {
      d.ancestor = d.address;
      continue;
    }
    for (int guard = 0; guard < 64; ++guard) {
      const auto up = parent_of.find(at);
      if (children[at] != 1 || up == parent_of.end() || up->second.empty()) break;
      at = up->second;
    }
    d.ancestor = at;
  }
  return devices;
}

std::vector<PciGpuPlacement> place_gpus(const std::vector<PciDevice>& devices,
                                        const std::vector<std::string>& gpu_addresses) {
  std::map<std::string, const PciDevice*> by_address;
  for (const PciDevice& d : devices) by_address[d.address] = &d;

  // RDMA-capable network functions; keep the most common model (a management NIC of another
  // make must not be handed to a GPU)
  std::map<std::pair<uint32_t, uint32_t>, int> model_count;
  for (const PciDevice& d : devices) {
    if ((d.pci_class >> 16) == 0x02 && !d.rdma_names.empty()) ++model_count[{d.vendor, d.device}];
  }
  std::pair<uint32_t, uint32_t> model{0, 0};
  int best = 0;
  for (const auto& [m, n] : model_count) {
    if (n > best) {
      best = n;
      model = m;
    }
  }

  struct Switch {
    std::vector<std::string> gpus;
    std::vector<const PciDevice*> nics;
  };
  std::map<std::string, Switch> switches;
  for (const std::string& g : gpu_addresses) {
    const auto it = by_address.find(g);
    if (it != by_address.end()) switches[it->second->ancestor].gpus.push_back(g);
  }
  if (best > 0) {
    for (const PciDevice& d : devices) {
      if ((d.pci_class >> 16) != 0x02 || d.rdma_names.empty()) continue;
      if (std::make_pair(d.vendor, d.device) != model) continue;
      const auto sw = switches.find(d.ancestor);
      if (sw != switches.end()) sw->second.nics.push_back(&d);
    }
  }

  std::vector<PciGpuPlacement> out;
  for (const std::string& g : gpu_addresses) {
    PciGpuPlacement p;
    p.gpu_address = g;
    const auto it = by_address.find(g);
    if (it != by_address.end()) {
      p.numa = it->second->numa;
      p.pci_switch = it->second->ancestor;
      const Switch& sw = switches[p.pci_switch];
      const size_t index = static_cast<size_t>(std::find(sw.gpus.begin(), sw.gpus.end(), g) - sw.gpus.begin());
      const size_t per_gpu = sw.nics.size() / sw.gpus.size();
      for (size_t i = index * per_gpu; i < (index + 1) * per_gpu; ++i) {
        const PciDevice* nic = sw.nics[i];
        p.nics.push_back(PciNic{nic->address, nic->rdma_names.empty() ? nic->address : nic->rdma_names.front()});
      }
    }
    out.push_back(std::move(p));
  }
  return out;
}

}  // namespace pplx::fabric
