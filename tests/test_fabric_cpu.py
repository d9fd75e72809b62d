"""Transfer engine on host memory (no GPU): types, sharding arithmetic, one-sided writes,
paged writes, immediates and counters, two-sided messages, scalar watchers, failure
reporting; inside one process and between two processes. The scenarios follow the
reference's tests/fabric_lib/test_transfer_engine.py:405-864, test_handle.py:13 and
test_types.py:4, which need four GPUs and RDMA NICs there."""

from __future__ import annotations

import ctypes
import multiprocessing as mp
import pickle
import threading
import time

import pytest
import torch

from pplx_garden import _native
from pplx_garden.fabric_lib import (
    DomainAddress,
    MemoryRegionDescriptor,
    PageIndices,
    ScatterTarget,
    TransferCounter,
    TransferEngine,
)


class Waiter:
    def __init__(self) -> None:
        self.event = threading.Event()
        self.errors: list[str] = []

    def done(self) -> None:
        self.event.set()

    def error(self, msg: str) -> None:
        self.errors.append(msg)
        self.event.set()

    def wait(self, timeout: float = 10.0) -> None:
        assert self.event.wait(timeout), "transfer did not complete in time"
        assert not self.errors, self.errors


@pytest.fixture()
def pair():
    a = TransferEngine(2, [-1])
    b = TransferEngine(2, [-1])
    yield a, b
    a.stop()
    b.stop()


def test_domain_address_value_semantics() -> None:
    a = DomainAddress.from_bytes(b"\x01\x02\xff")
    b = DomainAddress.from_str("0102ff")
    assert a == b and hash(a) == hash(b) and str(a) == "0102ff"
    assert a != DomainAddress.from_bytes(b"\x01\x02") and a != "0102ff"
    assert len({a, b}) == 1 and pickle.loads(pickle.dumps(a)) == a
    with pytest.raises(ValueError):
        DomainAddress.from_str("xyz")


def test_descriptor_round_trips(pair) -> None:
    a, _ = pair
    buf = torch.zeros(8192, dtype=torch.uint8)
    handle, desc = a.register_tensor(buf)
    again = MemoryRegionDescriptor.from_bytes(desc.as_bytes())
    assert again.as_bytes() == desc.as_bytes() and again.ptr == buf.data_ptr()
    assert pickle.loads(pickle.dumps(desc)).as_bytes() == desc.as_bytes()
    assert len(desc.addresses) == a.nets_per_gpu == 2 and desc.addresses[0] == a.main_address
    assert "MemoryRegionHandle" in handle.debug_str() and "0x" in desc.debug_str()
    with pytest.raises(ValueError):
        MemoryRegionDescriptor.from_bytes(b"junk")


def test_sharding_arithmetic() -> None:
    shard = _native._shard_single_transfer
    assert shard(100, 2) == [(0, 100), (0, 0)]              # a zero-length shard sits at offset 0
    assert shard(16384, 2) == [(0, 8192), (8192, 8192)]
    assert shard(16385, 2) == [(0, 8192), (8192, 8193)]     # no byte is lost to rounding
    assert shard(0, 3) == [(0, 0)] * 3
    for total in (1, 8191, 8192, 8193, 100_000, 1 << 20, (1 << 20) + 5):
        for n in (1, 2, 3, 4):
            parts = shard(total, n)
            assert len(parts) == n and sum(l for _, l in parts) == total
            pos = 0
            for off, length in parts:
                if length:
                    assert off == pos
                    pos += length
    pages = _native._shard_pages
    assert pages(10, 4) == [(0, 3), (3, 6), (6, 8), (8, 10)]
    assert pages(2, 4) == [(0, 1), (1, 2)] and pages(0, 4) == []
    assert _native._parse_cpu_list("0-3,8,10-11\n") == [0, 1, 2, 3, 8, 10, 11]
    assert _native._split_evenly(list(range(10)), 3, 0) == [0, 1, 2, 3]
    assert _native._split_evenly(list(range(10)), 3, 2) == [7, 8, 9]


def test_topology_has_a_group_per_device() -> None:
    topo = TransferEngine.detect_topology()
    assert topo and all(g.domains and g.cpus for g in topo)
    assert all(d.link_speed > 0 and d.name for g in topo for d in g.domains)


def test_single_write_all_shard_counts(pair) -> None:
    a, b = pair
    src = torch.randint(0, 255, (1 << 20,), dtype=torch.uint8)
    dst = torch.zeros(1 << 20, dtype=torch.uint8)
    hs, _ = a.register_tensor(src)
    _, dd = b.register_tensor(dst)
    for shards in (None, 1, 2):
        dst.zero_()
        w = Waiter()
        a.submit_write(hs, 4096, 300_000, None, dd, 8192, w.done, w.error, shards)
        w.wait()
        assert torch.equal(dst[8192:8192 + 300_000], src[4096:4096 + 300_000])
        assert dst[:8192].sum() == 0 and dst[8192 + 300_000:].sum() == 0
    w = Waiter()
    a.submit_write(hs, 0, 16, None, dd, 0, w.done, w.error, 3)      # more shards than domains
    assert w.event.wait(5) and w.errors and "num_shards" in w.errors[0]


def test_write_at_the_very_end_of_a_region(pair) -> None:
    """A short write split over two domains leaves one zero-length shard; it must not be
    issued at an offset past the region (reference regression test :762)."""
    a, b = pair
    src = torch.full((4096,), 7, dtype=torch.uint8)
    dst = torch.zeros(4096, dtype=torch.uint8)
    hs, _ = a.register_tensor(src)
    _, dd = b.register_tensor(dst)
    w = Waiter()
    a.submit_write(hs, 4096 - 64, 64, None, dd, 4096 - 64, w.done, w.error)
    w.wait()
    assert dst[-64:].eq(7).all() and dst[:-64].sum() == 0


def test_out_of_bounds_write_is_an_error(pair) -> None:
    a, b = pair
    src = torch.zeros(8192, dtype=torch.uint8)
    dst = torch.zeros(4096, dtype=torch.uint8)
    hs, _ = a.register_tensor(src)
    _, dd = b.register_tensor(dst)
    w = Waiter()
    a.submit_write(hs, 0, 8192, None, dd, 0, w.done, w.error, 1)
    assert w.event.wait(5) and w.errors and "past the end" in w.errors[0]


def test_out_of_bounds_source_is_an_error(pair) -> None:
    """The source side is range-checked on the host too: an offset, a page index or a stride
    that leaves the registered source region ends in the error callback and copies nothing."""
    a, b = pair
    src = torch.full((4096,), 5, dtype=torch.uint8)
    dst = torch.zeros(16384, dtype=torch.uint8)
    hs, _ = a.register_tensor(src)
    _, dd = b.register_tensor(dst)
    w = Waiter()
    a.submit_write(hs, 4096 - 32, 64, None, dd, 0, w.done, w.error, 1)          # offset + length
    assert w.event.wait(5) and w.errors and "source region" in w.errors[0]
    w = Waiter()
    a.submit_paged_writes(1024, hs, PageIndices([0, 4]), 1024, 0, dd, PageIndices([0, 1]), 1024, 0,
                          None, w.done, w.error)                                # page index
    assert w.event.wait(5) and w.errors and "source region" in w.errors[0]
    w = Waiter()
    a.submit_paged_writes(1024, hs, PageIndices([1]), 1 << 63, 0, dd, PageIndices([0]), 1024, 0,
                          None, w.done, w.error)                                # stride overflow
    assert w.event.wait(5) and w.errors
    # pages are spread over the domains: the valid page of the second request may have been
    # copied by its domain, nothing else
    assert int(dst[1024:].count_nonzero()) == 0


def test_paged_write_with_counted_immediates(pair) -> None:
    a, b = pair
    page, n_pages = 4096, 64
    src = torch.randint(0, 255, (n_pages * page,), dtype=torch.uint8)
    dst = torch.zeros(2 * n_pages * page, dtype=torch.uint8)
    hs, _ = a.register_tensor(src)
    _, dd = b.register_tensor(dst)
    src_pages = list(range(0, n_pages, 2))
    dst_pages = [n_pages - 1 - p for p in src_pages]
    reached = threading.Event()
    assert b.set_imm_count_expected(0x51, len(src_pages), reached.set) is None
    w = Waiter()
    a.submit_paged_writes(page // 2, hs, PageIndices(src_pages), page, 16, dd, PageIndices(dst_pages),
                          2 * page, 32, 0x51, w.done, w.error)
    w.wait()
    assert reached.wait(5), "every page must count as one immediate at the receiver"
    for s, d in zip(src_pages, dst_pages):
        assert torch.equal(dst[d * 2 * page + 32: d * 2 * page + 32 + page // 2],
                           src[s * page + 16: s * page + 16 + page // 2])
    assert int(dst.count_nonzero()) <= len(src_pages) * page // 2


def test_immediates_counters_and_surplus(pair) -> None:
    """Uncounted immediates go to the callback; an expected count consumes exactly that
    many arrivals and later ones fall through to the callback again (reference :784-845)."""
    a, b = pair
    buf = torch.zeros(4096, dtype=torch.uint8)
    _, dd = b.register_tensor(buf)
    seen: list[int] = []
    lock = threading.Lock()

    def on_imm(imm: int) -> None:
        with lock:
            seen.append(imm)

    b.set_imm_callback(on_imm)
    reached = threading.Event()
    b.set_imm_count_expected(5, 3, reached.set)
    waiters = []
    for imm in (5, 9, 5, 5, 5, 5):
        w = Waiter()
        a.submit_imm(imm, dd, w.done, w.error)
        waiters.append(w)
    for w in waiters:
        w.wait()
    assert reached.wait(5)
    deadline = time.time() + 5
    while time.time() < deadline and len(seen) < 3:
        time.sleep(0.01)
    assert sorted(seen) == [5, 5, 9]
    assert b.remove_imm_count(5) == (3, 3)
    assert b.remove_imm_count(5) is None
    counter = b.get_imm_counter(77)
    for _ in range(4):
        a.submit_imm(77, dd, lambda: None, lambda e: None)
    assert counter.wait(4, 5000) and not counter.wait(1, 50)


def test_two_sided_messages(pair) -> None:
    a, b = pair
    got: list[bytes] = []
    done = threading.Event()

    def on_recv(data: bytes) -> None:
        got.append(data)
        if len(got) == 5:
            done.set()

    b.submit_bouncing_recvs(2, 256, on_recv, lambda e: got.append(e.encode()))
    for i in range(5):                               # more messages than posted buffers: they are re-posted
        a.submit_send(b.main_address, f"message {i}".encode(), lambda: None, lambda e: None)
    assert done.wait(5) and sorted(got) == [f"message {i}".encode() for i in range(5)]


def test_scatter_and_barrier(pair) -> None:
    a, b = pair
    c = TransferEngine(2, [-1])
    try:
        src = torch.arange(64 * 1024, dtype=torch.int32)
        d1 = torch.zeros(32 * 1024, dtype=torch.int32)
        d2 = torch.zeros(32 * 1024, dtype=torch.int32)
        hs, _ = a.register_tensor(src)
        _, dd1 = b.register_tensor(d1)
        _, dd2 = c.register_tensor(d2)
        for routing in ("shard_peers", "shard_bytes", "single"):
            d1.zero_(); d2.zero_()
            w = Waiter()
            a.submit_scatter(hs, [ScatterTarget(dd1, 100_000, 0, 16), ScatterTarget(dd2, 64, 128 * 1024, 0)],
                             None, w.done, w.error, routing)
            w.wait()
            assert torch.equal(d1.view(torch.uint8)[16:100_016], src.view(torch.uint8)[:100_000])
            assert torch.equal(d2.view(torch.uint8)[:64], src.view(torch.uint8)[128 * 1024:128 * 1024 + 64])
        hits: list[int] = []
        b.set_imm_callback(hits.append)
        c.set_imm_callback(hits.append)
        w = Waiter()
        a.submit_barrier(0xB0, [dd1, dd2], w.done, w.error)
        w.wait()
        deadline = time.time() + 5
        while time.time() < deadline and len(hits) < 2:
            time.sleep(0.01)
        assert hits == [0xB0, 0xB0]
    finally:
        c.stop()


def test_atomic_submission_counts_completions_and_errors(pair) -> None:
    a, b = pair
    src = torch.ones(4096, dtype=torch.uint8)
    dst = torch.zeros(4096, dtype=torch.uint8)
    hs, _ = a.register_tensor(src)
    _, dd = b.register_tensor(dst)
    counter = TransferCounter()
    a._inject_write_failure(-1, 1)          # the next write on the first domain fails
    a.submit_write_atomic(hs, 0, 4096, None, dd, 0, counter)
    deadline = time.time() + 5
    while time.time() < deadline and counter.done < 1:
        time.sleep(0.001)
    assert counter.done == 1 and counter.errors == 1, "one shard failed: the transfer counts as an error"


def test_injected_failure_reaches_on_error(pair) -> None:
    a, b = pair
    src = torch.ones(4096, dtype=torch.uint8)
    dst = torch.zeros(4096, dtype=torch.uint8)
    hs, _ = a.register_tensor(src)
    _, dd = b.register_tensor(dst)
    a._inject_write_failure(-1, 1)
    w = Waiter()
    a.submit_write(hs, 0, 4096, None, dd, 0, w.done, w.error, 1)
    assert w.event.wait(5) and w.errors == ["injected write failure"]
    w = Waiter()                                          # the engine keeps working afterwards
    a.submit_write(hs, 0, 4096, None, dd, 0, w.done, w.error, 1)
    w.wait()
    assert dst.eq(1).all()


def test_scalar_watcher_sees_changes_and_can_stop(pair) -> None:
    a, _ = pair
    changes: list[tuple[int, int]] = []
    got_two = threading.Event()

    def on_change(old: int, new: int) -> bool:
        changes.append((old, new))
        if len(changes) == 2:
            got_two.set()
        return len(changes) < 2           # stop watching after the second change

    watcher = a.alloc_scalar_watcher(on_change)
    cell = ctypes.c_uint64.from_address(watcher.ptr)
    cell.value = 5
    time.sleep(0.05)
    cell.value = 9
    assert got_two.wait(5)
    time.sleep(0.05)
    cell.value = 11                        # released: no further callback
    time.sleep(0.1)
    assert changes == [(0, 5), (5, 9)]


def test_unregistered_source_and_stopped_engine() -> None:
    a = TransferEngine(1, [-1])
    b = TransferEngine(1, [-1])
    try:
        buf = torch.zeros(4096, dtype=torch.uint8)
        h, d = b.register_tensor(buf)
        with pytest.raises(ValueError, match="not registered"):
            a.submit_write(h, 0, 16, None, d, 0, lambda: None, lambda e: None)
    finally:
        a.stop()
        b.stop()
    with pytest.raises(RuntimeError, match="stopped|down"):
        a.register_tensor(torch.zeros(16, dtype=torch.uint8))


# ---- two processes ---------------------------------------------------------

def _server(conn) -> None:
    engine = TransferEngine(1, [-1])
    buf = torch.zeros(1 << 16, dtype=torch.uint8)
    _, desc = engine.register_tensor(buf)
    reached = threading.Event()
    engine.set_imm_count_expected(3, 4, reached.set)
    requests: list[bytes] = []
    got = threading.Event()
    engine.submit_bouncing_recvs(1, 128, lambda d: (requests.append(d), got.set()), lambda e: None)
    conn.send((engine.main_address.as_bytes(), desc.as_bytes()))
    ok = reached.wait(20) and got.wait(20)
    conn.send((ok, bytes(buf[:8].tolist()), bytes(buf[3 * 4096: 3 * 4096 + 4].tolist()), requests))
    engine.stop()


def test_writes_and_messages_between_processes() -> None:
    ctx = mp.get_context("spawn")
    parent, child = ctx.Pipe()
    proc = ctx.Process(target=_server, args=(child,))
    proc.start()
    try:
        addr_bytes, desc_bytes = parent.recv()
        engine = TransferEngine(1, [-1])
        src = (torch.arange(1 << 16) % 251).to(torch.uint8)
        handle, _ = engine.register_tensor(src)
        desc = MemoryRegionDescriptor.from_bytes(desc_bytes)
        w = Waiter()
        engine.submit_paged_writes(4096, handle, PageIndices([0, 1, 2, 3]), 4096, 0, desc,
                                   PageIndices([0, 1, 2, 3]), 4096, 0, 3, w.done, w.error)
        w.wait(20)
        s = Waiter()
        engine.submit_send(DomainAddress.from_bytes(addr_bytes), b"ping", s.done, s.error)
        s.wait(20)
        ok, head, third, requests = parent.recv()
        assert ok and head == bytes(src[:8].tolist()) and third == bytes(src[3 * 4096: 3 * 4096 + 4].tolist())
        assert requests == [b"ping"]
        engine.stop()
    finally:
        proc.join(20)
        if proc.is_alive():
            proc.terminate()


def _fake_pci(root, path, vendor, device, pci_class, numa, rdma=None):
    """One PCI function in a fake sysfs: `path` is the chain of addresses below the root complex."""
    import os

    real = os.path.join(root, "devices", "pci0000:00", *path)
    os.makedirs(real, exist_ok=True)
    for name, value in (("vendor", f"0x{vendor:04x}"), ("device", f"0x{device:04x}"),
                        ("class", f"0x{pci_class:06x}"), ("numa_node", str(numa))):
        with open(os.path.join(real, name), "w") as f:
            f.write(value + "\n")
    if rdma:
        os.makedirs(os.path.join(real, "infiniband", rdma))
    link_dir = os.path.join(root, "bus", "pci", "devices")
    os.makedirs(link_dir, exist_ok=True)
    link = os.path.join(link_dir, path[-1])
    if not os.path.lexists(link):
        os.symlink(real, link)


def test_pci_placement_groups_gpus_and_nics_by_switch(tmp_path) -> None:
    """Two PCIe switches, each with two GPUs and two NICs behind single-child bridges, plus a NIC
    of another make next to the root: every GPU gets the NIC share of its own switch
    (reference fabric-lib/src/topo.rs:285-458)."""
    from pplx_garden import _native

    root = str(tmp_path)
    bridge, gpu, nic = 0x060400, 0x030200, 0x020700
    for sw, bus in ((0, 0x10), (1, 0x40)):
        up = f"0000:{bus:02x}:00.0"                       # root port
        switch = f"0000:{bus + 1:02x}:00.0"               # switch upstream port
        _fake_pci(root, [up], 0x8086, 0x1, bridge, sw)
        _fake_pci(root, [up, switch], 0x1000, 0x2, bridge, sw)
        for i in range(4):                                # four downstream ports
            down = f"0000:{bus + 2:02x}:{i:02x}.0"
            _fake_pci(root, [up, switch, down], 0x1000, 0x3, bridge, sw)
            leaf = f"0000:{bus + 3 + i:02x}:00.0"
            if i < 2:
                _fake_pci(root, [up, switch, down, leaf], 0x10de, 0x2901, gpu, sw)
            else:
                _fake_pci(root, [up, switch, down, leaf], 0x15b3, 0x1021, nic, sw, rdma=f"mlx5_{2 * sw + i - 2}")
    _fake_pci(root, ["0000:00:1f.0"], 0x8086, 0x9, bridge, 0)
    _fake_pci(root, ["0000:00:1f.0", "0000:05:00.0"], 0x14e4, 0x1750, 0x020000, 0, rdma="bnxt_re0")

    gpus = ["0000:13:00.0", "0000:14:00.0", "0000:43:00.0", "0000:44:00.0"]
    placed = _native._place_gpus_from_sysfs(root, gpus + ["0000:99:00.0"])
    assert [p[0] for p in placed] == gpus + ["0000:99:00.0"]
    assert placed[0][1] == placed[1][1] == "0000:11:00.0"      # the switch, not the single-child port above it
    assert placed[2][1] == placed[3][1] == "0000:41:00.0"
    assert [p[2] for p in placed[:4]] == [0, 0, 1, 1]
    assert [[n[1] for n in p[3]] for p in placed[:4]] == [["mlx5_0"], ["mlx5_1"], ["mlx5_2"], ["mlx5_3"]]
    assert placed[4][1] == "" and placed[4][3] == []             # unknown GPU: no switch, no NICs


def test_topology_reports_pci_fields() -> None:
    from pplx_garden.fabric_lib import TransferEngine

    for group in TransferEngine.detect_topology():
        assert isinstance(group.pci_address, str) and isinstance(group.pci_switch, str)
        assert isinstance(group.nics, list)
        assert group.domains and group.domains[0].link_speed > 0


def test_fault_decorator_drop_delay_reorder(pair) -> None:
    """Host-side fault injection on the provider seam: a dropped write never completes, a delayed
    one completes late with its bytes in place, reordered completions arrive newest first, and the
    engine is back to normal once the faults are cleared."""
    import time

    a, b = pair
    src = torch.arange(4096, dtype=torch.int32).view(torch.uint8).clone()
    dst = torch.zeros_like(src)
    hs, _ = a.register_tensor(src)
    _, dd = b.register_tensor(dst)

    # drop: neither callback fires; a later write is unaffected
    a._inject_fault(-1, "drop", 1)
    lost = Waiter()
    a.submit_write(hs, 0, 64, None, dd, 0, lost.done, lost.error, 1)
    ok = Waiter()
    a.submit_write(hs, 64, 64, None, dd, 64, ok.done, ok.error, 1)
    ok.wait()
    assert not lost.event.wait(0.3) and not lost.errors
    assert dst[:64].sum() == 0 and torch.equal(dst[64:128], src[64:128])

    # delay: completion is held back, data is already there
    a._inject_fault(-1, "delay", 300)
    late = Waiter()
    t0 = time.monotonic()
    a.submit_write(hs, 128, 64, None, dd, 128, late.done, late.error, 1)
    late.wait()
    assert time.monotonic() - t0 >= 0.25
    assert torch.equal(dst[128:192], src[128:192])
    a._inject_fault(-1, "none")

    # reorder: writes alternate between the engine's two domains; on each, a batch of two
    # completes newest first
    for domain in range(a.nets_per_gpu):
        a._inject_fault(-1, "reorder", 2, domain)
    order: list[int] = []
    waiters = []
    for i in range(2 * a.nets_per_gpu):
        w = Waiter()
        waiters.append(w)
        a.submit_write(hs, 256 + 64 * i, 64, None, dd, 256 + 64 * i,
                       (lambda i=i, w=w: (order.append(i), w.done())), w.error, 1)
    for w in waiters:
        w.wait()
    n = a.nets_per_gpu
    for first in range(n):
        assert order.index(first + n) < order.index(first), order
    for domain in range(a.nets_per_gpu):
        a._inject_fault(-1, "none", 0, domain)
    a._inject_fault(-1, "none")
    last = Waiter()
    a.submit_write(hs, 1024, 64, None, dd, 1024, last.done, last.error, 1)
    last.wait()
    assert torch.equal(dst[1024:1088], src[1024:1088])
