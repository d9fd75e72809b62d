// PCI tree of the machine, read from sysfs: which GPUs sit under the same PCIe switch and
// which RDMA-capable NICs sit there with them.
//
// Behaviour follows the reference's fabric-lib/src/topo.rs:285-381 ("branching ancestor":
// from a device walk up through bridges that have a single child; devices that end at the
// same ancestor share a switch) and :391-458 (the NICs of a switch are dealt out evenly to
// its GPUs). The scan takes the sysfs root as an argument so that it can be tested against a
// directory tree built by a test.
#pragma once

#include <cstdint>
#include <map>
#include <string>
#include <vector>

namespace pplx::fabric {

struct PciDevice {
  std::string address;    // "0000:1b:00.0"
  std::string parent;     // enclosing bridge, empty for a device directly under a root complex
  std::string ancestor;   // branching ancestor (see above); a root-level device is its own
  uint32_t vendor = 0, device = 0, pci_class = 0;
  int numa = -1;
  std::vector<std::string> rdma_names;  // entries of <device>/infiniband/, e.g. "mlx5_0"
};

// Every PCI function below `<sysfs_root>/bus/pci/devices`, sorted by address, with parents and
// branching ancestors filled in. A missing directory gives an empty list.
std::vector<PciDevice> scan_pci(const std::string& sysfs_root);

struct PciNic {
  std::string address;
  std::string name;  // RDMA device name when the driver exposes one, else the PCI address
};

struct PciGpuPlacement {
  std::string gpu_address;
  std::string pci_switch;     // branching ancestor shared with the NICs below
  int numa = -1;
  std::vector<PciNic> nics;   // this GPU's share of the switch's NICs
};

// Places the GPUs with the given PCI addresses (lower case, as in sysfs). NICs are the
// RDMA-capable network functions (class 0x02, with an infiniband/ directory) of the most common
// (vendor, device) pair; a switch with g GPUs and n such NICs gives each GPU n / g of them, in
// address order. GPUs that the scan did not find are returned with empty switch and no NICs.
std::vector<PciGpuPlacement> place_gpus(const std::vector<PciDevice>& devices,
                                        const std::vector<std::string>& gpu_addresses);

}  // namespace pplx::fabric
