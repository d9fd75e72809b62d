// Machine topology for placing transfer-engine threads: which NUMA node and CPU cores sit
// next to each GPU, and which transport domains serve it.
// Reference: fabric-lib/src/topo.rs:158-550 (sysfs PCI walk, NUMA-local physical cores
// split evenly between the GPUs of a node, NICs grouped with the GPU under the same PCIe
// switch). Without RDMA NICs every GPU gets the intra-box NVLink domain.
#pragma once

#include <string>
#include <vector>

#include "provider.h"

namespace pplx::fabric {

struct TopologyGroup {
  int cuda_device = -1;          // -1: host-only group (machine without a GPU)
  int numa = 0;
  std::vector<DomainInfo> domains;
  std::vector<int> cpus;         // physical cores near the device, in preference order
};

// Cached after the first call. Never throws: missing sysfs entries degrade to "NUMA 0,
// all CPUs of the process".
const std::vector<TopologyGroup>& detect_topology();

// Pure helpers (unit tested): "0-3,8,10-11" -> {0,1,2,3,8,10,11}
std::vector<int> parse_cpu_list(const std::string& text);
// Splits `cpus` into `parts` nearly equal consecutive slices and returns slice `index`.
std::vector<int> split_evenly(const std::vector<int>& cpus, size_t parts, size_t index);

}  // namespace pplx::fabric
