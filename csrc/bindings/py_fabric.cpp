// Python bindings of the transfer engine: the classes and methods of the reference's
// python-ext/src/py_fabric_lib.rs:35-735 (typed in pplx_garden/fabric_lib.pyi), plus the
// scatter / barrier submissions and the atomic (counter based) variants that the reference
// keeps Rust-only (fabric-lib/src/api.rs:122-175).
//
// Python callbacks run on the engine's callback thread; pybind11's std::function caster
// takes the GIL around each call. Every method that may block on an engine thread releases
// the GIL first.
#include <pybind11/functional.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include "../core/error.h"
#include "../fabric/faulty_domain.h"
#include "../fabric/local_domain.h"
#include "../fabric/shard.h"
#include "../fabric/transfer_engine.h"
#include "py_fabric.h"
#include "py_util.h"

namespace py = pybind11;
using namespace pplx;
using namespace pplx::fabric;

namespace {

struct PyPageIndices {
  std::shared_ptr<const std::vector<uint32_t>> pages;
};

struct PyBuilder {
  TransferEngineBuilder builder;
};

std::vector<GpuDomainSpec> specs_from_topology(size_t nets_per_gpu, const std::vector<int>& devices) {
  const auto& topo = detect_topology();
  std::vector<GpuDomainSpec> out;
  for (int dev : devices) {
    const TopologyGroup* g = nullptr;
    for (const auto& t : topo) {
      if (t.cuda_device == dev) g = &t;
    }
    if (g == nullptr) throw Error(ErrorKind::kInvalidArgument, "cuda:" + std::to_string(dev) + " is not in the detected topology");
    GpuDomainSpec spec;
    spec.cuda_device = dev;
    for (size_t i = 0; i < std::max<size_t>(nets_per_gpu, 1); ++i) {
      // the intra-box provider can open as many copy queues per GPU as asked for
      DomainInfo info = g->domains[std::min(i, g->domains.size() - 1)];
      if (i >= g->domains.size()) info.name = "nvl" + std::to_string(i) + ":cuda" + std::to_string(dev);
      spec.domains.push_back(info);
    }
    spec.pin_worker_cpu = g->cpus.size() > 1 ? g->cpus[1] : -1;
    spec.pin_uvm_cpu = g->cpus.size() > 2 ? g->cpus[2] : -1;
    out.push_back(std::move(spec));
  }
  return out;
}

DomainGroupRouting routing_from(const py::object& num_shards, size_t nets) {
  if (num_shards.is_none()) return DomainGroupRouting::sharded(static_cast<uint8_t>(std::max<size_t>(nets, 1)));
  return DomainGroupRouting::sharded(num_shards.cast<uint8_t>());
}

std::optional<uint32_t> opt_imm(const py::object& imm) {
  if (imm.is_none()) return std::nullopt;
  return imm.cast<uint32_t>();
}

}  // namespace

void bind_fabric(py::module_& m) {
  py::class_<DomainInfo>(m, "DomainInfo")
      .def_property_readonly("name", [](const DomainInfo& d) { return d.name; })
      .def_property_readonly("link_speed", [](const DomainInfo& d) { return d.link_speed; })
      .def_property_readonly("provider", [](const DomainInfo& d) { return d.provider; })
      .def("__repr__", [](const DomainInfo& d) {
        return "DomainInfo(name='" + d.name + "', link_speed=" + std::to_string(d.link_speed) + ")";
      });

  py::class_<DomainAddress>(m, "DomainAddress")
      .def_static("from_bytes", [](const py::bytes& b) { return DomainAddress(std::string(b)); }, py::arg("bytes"))
      .def("as_bytes", [](const DomainAddress& a) { return py::bytes(a.bytes()); })
      .def_static("from_str", [](const std::string& s) { return DomainAddress::from_hex(s); })
      .def("__str__", &DomainAddress::to_hex)
      .def("__repr__", [](const DomainAddress& a) { return "DomainAddress(" + a.to_hex() + ")"; })
      .def("__eq__", [](const DomainAddress& a, const py::object& o) {
        return py::isinstance<DomainAddress>(o) && a == o.cast<DomainAddress>();
      })
      .def("__hash__", &DomainAddress::hash)
      .def(py::pickle([](const DomainAddress& a) { return py::bytes(a.bytes()); },
                      [](const py::bytes& b) { return DomainAddress(std::string(b)); }));

  py::class_<TopologyGroup>(m, "TopologyGroup")
      .def_property_readonly("cuda_device", [](const TopologyGroup& g) { return g.cuda_device; })
      .def_property_readonly("numa", [](const TopologyGroup& g) { return g.numa; })
      .def_property_readonly("domains", [](const TopologyGroup& g) { return g.domains; })
      .def_property_readonly("cpus", [](const TopologyGroup& g) { return g.cpus; })
      .def_property_readonly("pci_address", [](const TopologyGroup& g) { return g.pci_address; })
      .def_property_readonly("pci_switch", [](const TopologyGroup& g) { return g.pci_switch; })
      .def_property_readonly("nics", [](const TopologyGroup& g) { return g.nics; });
  m.def(
      "_place_gpus_from_sysfs",
      [](const std::string& sysfs_root, const std::vector<std::string>& gpu_addresses) {
        py::list out;
        for (const PciGpuPlacement& p : place_gpus(scan_pci(sysfs_root), gpu_addresses)) {
          py::list nics;
          for (const PciNic& n : p.nics) nics.append(py::make_tuple(n.address, n.name));
          out.append(py::make_tuple(p.gpu_address, p.pci_switch, p.numa, nics));
        }
        return out;
      },
      py::arg("sysfs_root"), py::arg("gpu_addresses"),
      "PCI placement of GPUs (switch, NUMA node, share of the switch's RDMA NICs) from a sysfs tree.");

  py::class_<MemoryRegionHandle>(m, "MemoryRegionHandle")
      .def_property_readonly("ptr", [](const MemoryRegionHandle& h) { return h.ptr; })
      .def("capsule", [](const MemoryRegionHandle& h) {
        return py::capsule(reinterpret_cast<void*>(h.ptr), "pplx_garden.MemoryRegionHandle");
      })
      .def("debug_str", [](const MemoryRegionHandle& h) {
        char buf[64];
        std::snprintf(buf, sizeof(buf), "MemoryRegionHandle(ptr=0x%llx)", static_cast<unsigned long long>(h.ptr));
        return std::string(buf);
      });

  py::class_<MemoryRegionDescriptor>(m, "MemoryRegionDescriptor")
      .def_static("from_bytes", [](const py::bytes& b) { return MemoryRegionDescriptor::deserialize(std::string(b)); },
                  py::arg("bytes_"))
      .def("as_bytes", [](const MemoryRegionDescriptor& d) { return py::bytes(d.serialize()); })
      .def("debug_str", &MemoryRegionDescriptor::debug_str)
      .def_property_readonly("ptr", [](const MemoryRegionDescriptor& d) { return d.ptr; })
      .def_property_readonly("addresses", [](const MemoryRegionDescriptor& d) {
        std::vector<DomainAddress> out;
        for (const auto& p : d.addr_rkey_list) out.push_back(p.first);
        return out;
      })
      .def(py::pickle([](const MemoryRegionDescriptor& d) { return py::bytes(d.serialize()); },
                      [](const py::bytes& b) { return MemoryRegionDescriptor::deserialize(std::string(b)); }));

  py::class_<PyPageIndices>(m, "PageIndices")
      .def(py::init([](const std::vector<uint32_t>& indices) {
             return PyPageIndices{std::make_shared<const std::vector<uint32_t>>(indices)};
           }),
           py::arg("indices"))
      .def("__len__", [](const PyPageIndices& p) { return p.pages->size(); });

  py::class_<UvmWatcher>(m, "UvmWatcher").def_property_readonly("ptr", &UvmWatcher::ptr);

  py::class_<ScatterTarget>(m, "ScatterTarget")
      .def(py::init([](const MemoryRegionDescriptor& dst_mr, uint64_t length, uint64_t src_offset, uint64_t dst_offset) {
             return ScatterTarget{dst_mr, length, src_offset, dst_offset};
           }),
           py::arg("dst_mr"), py::arg("length"), py::arg("src_offset"), py::arg("dst_offset"));

  py::class_<TransferCounter>(m, "TransferCounter")
      .def(py::init([] {
        return TransferCounter(std::make_shared<std::atomic<int64_t>>(0), std::make_shared<std::atomic<int64_t>>(0));
      }))
      .def_property_readonly("done", &TransferCounter::done)
      .def_property_readonly("errors", &TransferCounter::errors);

  py::class_<ImmCounter>(m, "ImmCounter")
      .def("wait", &ImmCounter::wait, py::arg("target"), py::arg("deadline_ms") = -1,
           py::call_guard<py::gil_scoped_release>())
      .def_property_readonly("value", &ImmCounter::value);

  py::class_<PyBuilder>(m, "TransferEngineBuilder")
      .def("add_gpu_domains",
           [](PyBuilder& b, int cuda_device, const std::vector<DomainInfo>& domains, int pin_worker_cpu,
              int pin_uvm_cpu) -> PyBuilder& {
             b.builder.add_gpu_domains(cuda_device, domains, pin_worker_cpu, pin_uvm_cpu);
             return b;
           },
           py::arg("cuda_device"), py::arg("domains"), py::arg("pin_worker_cpu"), py::arg("pin_uvm_cpu"),
           py::return_value_policy::reference_internal)
      .def("build", [](PyBuilder& b) {
        py::gil_scoped_release release;
        return PyEngine{b.builder.build()};
      });

  py::class_<PyEngine>(m, "TransferEngine")
      .def(py::init([](size_t nets_per_gpu, const std::vector<int>& cuda_devices) {
             py::gil_scoped_release release;
             return PyEngine{std::make_unique<TransferEngine>(specs_from_topology(nets_per_gpu, cuda_devices))};
           }),
           py::arg("nets_per_gpu"), py::arg("cuda_devices"))
      .def_static("detect_topology", [] { return detect_topology(); })
      .def_static("builder", [] { return PyBuilder{}; })
      .def_property_readonly("main_address", [](PyEngine& e) { return e.get().main_address(); })
      .def_property_readonly("num_domains", [](PyEngine& e) { return e.get().num_domains(); })
      .def_property_readonly("aggregated_link_speed", [](PyEngine& e) { return e.get().aggregated_link_speed(); })
      .def_property_readonly("nets_per_gpu", [](PyEngine& e) { return e.get().nets_per_gpu(); })
      .def_property_readonly("fabric_engine", [](py::object self) { return self; },
                             "The engine itself: the worker layer is not a separate Python object here.")
      .def("stop",
           [](PyEngine& e) {
             if (!e.engine) return;
             py::gil_scoped_release release;
             e.engine->stop();
           })
      .def("register_tensor",
           [](PyEngine& e, const py::object& tensor) {
             PPLX_REQUIRE(tensor.attr("is_contiguous")().cast<bool>(), "register_tensor needs a contiguous tensor");
             const uint64_t ptr = tensor.attr("data_ptr")().cast<uint64_t>();
             const uint64_t len = tensor.attr("numel")().cast<uint64_t>() * tensor.attr("element_size")().cast<uint64_t>();
             const int device = pplx_py::device_index(tensor.attr("device"), 0);
             TransferEngine& eng = e.get();
             py::gil_scoped_release release;
             return eng.register_memory(ptr, len, device);
           },
           py::arg("tensor"))
      .def("register_memory",
           [](PyEngine& e, uint64_t ptr, uint64_t len, const py::object& device) {
             const int dev = pplx_py::device_index(device, 0);
             TransferEngine& eng = e.get();
             py::gil_scoped_release release;
             return eng.register_memory(ptr, len, dev);
           },
           py::arg("ptr"), py::arg("len"), py::arg("device"))
      .def("unregister_memory",
           [](PyEngine& e, uint64_t ptr) {
             TransferEngine& eng = e.get();
             py::gil_scoped_release release;
             eng.unregister_memory(ptr);
           },
           py::arg("ptr"))
      .def("alloc_scalar_watcher",
           [](PyEngine& e, TransferEngine::WatchFn cb) { return e.get().alloc_scalar_watcher(std::move(cb)); },
           py::arg("callback"))
      .def("set_imm_callback", [](PyEngine& e, TransferEngine::ImmFn cb) { e.get().set_imm_callback(std::move(cb)); },
           py::arg("callback"))
      .def("set_imm_count_expected",
           [](PyEngine& e, uint32_t imm, uint32_t expected, TransferEngine::DoneFn cb) {
             return e.get().set_imm_count_expected(imm, expected, std::move(cb));
           },
           py::arg("imm"), py::arg("expected_count"), py::arg("on_reached"))
      .def("remove_imm_count", [](PyEngine& e, uint32_t imm) { return e.get().remove_imm_count(imm); }, py::arg("imm"))
      .def("get_imm_counter", [](PyEngine& e, uint32_t imm) { return e.get().get_imm_counter(imm); }, py::arg("imm"))
      .def("submit_bouncing_recvs",
           [](PyEngine& e, size_t count, size_t len, std::function<void(py::bytes)> on_recv,
              TransferEngine::ErrorFn on_error) {
             e.get().submit_bouncing_recvs(
                 count, len,
                 [on_recv = std::move(on_recv)](const std::string& data) {
                   py::gil_scoped_acquire gil;
                   on_recv(py::bytes(data));
                 },
                 std::move(on_error));
           },
           py::arg("count"), py::arg("len"), py::arg("on_recv"), py::arg("on_error"))
      .def("submit_send",
           [](PyEngine& e, const DomainAddress& addr, const py::bytes& data, TransferEngine::DoneFn on_done,
              TransferEngine::ErrorFn on_error) {
             std::string payload(data);
             TransferEngine& eng = e.get();
             py::gil_scoped_release release;
             eng.submit_send(addr, std::move(payload), std::move(on_done), std::move(on_error));
           },
           py::arg("addr"), py::arg("data"), py::arg("on_done"), py::arg("on_error"))
      .def("submit_imm",
           [](PyEngine& e, uint32_t imm, const MemoryRegionDescriptor& dst, TransferEngine::DoneFn on_done,
              TransferEngine::ErrorFn on_error) {
             ImmTransferRequest r{imm, dst, DomainGroupRouting::sharded(1)};
             TransferEngine& eng = e.get();
             py::gil_scoped_release release;
             eng.submit_transfer(std::move(r), std::move(on_done), std::move(on_error));
           },
           py::arg("imm_data"), py::arg("dst_mr"), py::arg("on_done"), py::arg("on_error"))
      .def("submit_write",
           [](PyEngine& e, const MemoryRegionHandle& src, uint64_t offset, uint64_t length, const py::object& imm,
              const MemoryRegionDescriptor& dst, uint64_t dst_offset, TransferEngine::DoneFn on_done,
              TransferEngine::ErrorFn on_error, const py::object& num_shards) {
             SingleTransferRequest r;
             r.src_mr = src;
             r.src_offset = offset;
             r.length = length;
             r.imm_data = opt_imm(imm);
             r.dst_mr = dst;
             r.dst_offset = dst_offset;
             r.domain = routing_from(num_shards, e.get().nets_per_gpu());
             TransferEngine& eng = e.get();
             py::gil_scoped_release release;
             eng.submit_transfer(std::move(r), std::move(on_done), std::move(on_error));
           },
           py::arg("src_mr"), py::arg("offset"), py::arg("length"), py::arg("imm_data"), py::arg("dst_mr"),
           py::arg("dst_offset"), py::arg("on_done"), py::arg("on_error"), py::arg("num_shards") = py::none())
      .def("submit_paged_writes",
           [](PyEngine& e, uint64_t length, const MemoryRegionHandle& src, const PyPageIndices& src_pages,
              uint64_t src_stride, uint64_t src_offset, const MemoryRegionDescriptor& dst,
              const PyPageIndices& dst_pages, uint64_t dst_stride, uint64_t dst_offset, const py::object& imm,
              TransferEngine::DoneFn on_done, TransferEngine::ErrorFn on_error) {
             PagedTransferRequest r;
             r.length = length;
             r.src_mr = src;
             r.src_page_indices = src_pages.pages;
             r.src_stride = src_stride;
             r.src_offset = src_offset;
             r.dst_mr = dst;
             r.dst_page_indices = dst_pages.pages;
             r.dst_stride = dst_stride;
             r.dst_offset = dst_offset;
             r.imm_data = opt_imm(imm);
             TransferEngine& eng = e.get();
             py::gil_scoped_release release;
             eng.submit_transfer(std::move(r), std::move(on_done), std::move(on_error));
           },
           py::arg("length"), py::arg("src_mr"), py::arg("src_page_indices"), py::arg("src_stride"),
           py::arg("src_offset"), py::arg("dst_mr"), py::arg("dst_page_indices"), py::arg("dst_stride"),
           py::arg("dst_offset"), py::arg("imm_data"), py::arg("on_done"), py::arg("on_error"))
      .def("submit_scatter",
           [](PyEngine& e, const MemoryRegionHandle& src, const std::vector<ScatterTarget>& targets,
              const py::object& imm, TransferEngine::DoneFn on_done, TransferEngine::ErrorFn on_error,
              const std::string& routing) {
             ScatterTransferRequest r;
             r.src_mr = src;
             r.dsts = std::make_shared<const std::vector<ScatterTarget>>(targets);
             r.imm_data = opt_imm(imm);
             if (routing == "shard_peers") r.domain.kind = GroupTransferRouting::Kind::kAllDomainsShardPeers;
             else if (routing == "shard_bytes") r.domain.kind = GroupTransferRouting::Kind::kAllDomainsShardBytes;
             else if (routing == "single") r.domain.kind = GroupTransferRouting::Kind::kSingle;
             else throw Error(ErrorKind::kInvalidArgument, "routing must be shard_peers, shard_bytes or single");
             TransferEngine& eng = e.get();
             py::gil_scoped_release release;
             eng.submit_transfer(std::move(r), std::move(on_done), std::move(on_error));
           },
           py::arg("src_mr"), py::arg("targets"), py::arg("imm_data"), py::arg("on_done"), py::arg("on_error"),
           py::arg("routing") = "shard_peers",
           "Fan one source region out to several destinations (weight shards, all-to-all ranges).")
      .def("submit_barrier",
           [](PyEngine& e, uint32_t imm, const std::vector<MemoryRegionDescriptor>& dsts,
              TransferEngine::DoneFn on_done, TransferEngine::ErrorFn on_error) {
             BarrierTransferRequest r{imm, dsts, DomainGroupRouting::pinned(0)};
             TransferEngine& eng = e.get();
             py::gil_scoped_release release;
             eng.submit_transfer(std::move(r), std::move(on_done), std::move(on_error));
           },
           py::arg("imm_data"), py::arg("dst_mrs"), py::arg("on_done"), py::arg("on_error"))
      .def("submit_write_atomic",
           [](PyEngine& e, const MemoryRegionHandle& src, uint64_t offset, uint64_t length, const py::object& imm,
              const MemoryRegionDescriptor& dst, uint64_t dst_offset, const TransferCounter& counter) {
             SingleTransferRequest r;
             r.src_mr = src;
             r.src_offset = offset;
             r.length = length;
             r.imm_data = opt_imm(imm);
             r.dst_mr = dst;
             r.dst_offset = dst_offset;
             r.domain = DomainGroupRouting::sharded(static_cast<uint8_t>(e.get().nets_per_gpu()));
             TransferEngine& eng = e.get();
             py::gil_scoped_release release;
             eng.submit_transfer_atomic(std::move(r), counter);
           },
           py::arg("src_mr"), py::arg("offset"), py::arg("length"), py::arg("imm_data"), py::arg("dst_mr"),
           py::arg("dst_offset"), py::arg("counter"))
      .def("_inject_write_failure",
           [](PyEngine& e, int device, uint64_t nth) {
             auto* d = dynamic_cast<FaultyDomain*>(e.get().debug_domain(device));
             PPLX_REQUIRE(d != nullptr, "this engine's domains are not behind the fault-injection decorator");
             d->inject(FaultKind::kFailWrite, nth);
           },
           py::arg("device"), py::arg("nth"), "Test hook: fail the n-th write submitted from now on.")
      .def("_inject_fault",
           [](PyEngine& e, int device, const std::string& kind, uint64_t value, size_t domain) {
             auto* d = dynamic_cast<FaultyDomain*>(e.get().debug_domain(device, domain));
             PPLX_REQUIRE(d != nullptr, "this engine's domains are not behind the fault-injection decorator");
             FaultKind k = FaultKind::kNone;
             if (kind == "fail") k = FaultKind::kFailWrite;
             else if (kind == "drop") k = FaultKind::kDropWrite;
             else if (kind == "delay") k = FaultKind::kDelayWrites;
             else if (kind == "reorder") k = FaultKind::kReorderWrites;
             else PPLX_REQUIRE(kind == "none", "fault kind must be fail, drop, delay, reorder or none");
             d->inject(k, value);
           },
           py::arg("device"), py::arg("kind"), py::arg("value") = 0, py::arg("domain") = 0,
           "Test hook on one domain of one device: 'fail' / 'drop' the value-th write from now, 'delay' write "
           "completions by value ms, 'reorder' them in batches of value (newest first), 'none' clears.");

  m.def("_shard_single_transfer", &shard_single_transfer, py::arg("total"), py::arg("num_shards"));
  m.def("_shard_pages", &shard_pages, py::arg("num_pages"), py::arg("num_shards"));
  m.def("_parse_cpu_list", &parse_cpu_list);
  m.def("_split_evenly", &split_evenly);
}
