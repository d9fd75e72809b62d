// Machine topology for placing transfer-engine threads: which NUMA node and CPU cores sit
// next to each GPU, and which transport domains serve it.
// Reference: fabric-lib/src/topo.rs:158-550 (sysfs PCI walk, NUMA-local physical cores
// split evenly between the GPUs of a node, NICs grouped with the GPU under the same PCIe
// switch). Without RDMA NICs every GPU gets the intra-box NVLink domain.
#pragma once

#include <string>
#include <vector>

#include "pci_topo.h"
#include "provider.h"

namespace pplx::fabric {

struct TopologyGroup {
  int cuda_device = -1;          // -1: host-only group (machine without a GPU)
  int numa = 0;
  std::vector<DomainInfo> domains;
  std::vector<int> cpus;         // physical cores near the device, in preference order
  std::string pci_address;       // of the GPU, lower case as in sysfs; empty when unknown
  std::string pci_switch;        // PCIe switch (branching ancestor) the GPU hangs off
  std::vector<DomainInfo> nics;  // RDMA NICs under the same switch, this GPU's share; they are
                                 // listed for placement only: no provider drives them here
};

// NVLink bandwidth of a GPU in bits per second and direction: active links x per-link speed as
// NVML reports them, or 0 when NVML cannot be asked.
uint64_t nvlink_bits_per_second(int cuda_device);

// Cached after the first call. Never throws: missing sysfs entries degrade to "NUMA 0,
// all CPUs of the process".
const std::vector<TopologyGroup>& detect_topology();

// Pure helpers (unit tested): "0-3,8,10-11" -> {0,1,2,3,8,10,11}
std::vector<int> parse_cpu_list(const std::string& text);
// Splits `cpus` into `parts` nearly equal consecutive slices and returns slice `index`.
std::vector<int> split_evenly(const std::vector<int>& cpus, size_t parts, size_t index);

}  // namespace pplx::fabric
