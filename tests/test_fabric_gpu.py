"""Transfer engine on GPU memory: the peer-copy kernel (bulk and SIMT paths), host<->device
writes, the scalar watcher driven by a kernel, and CUDA-IPC mapped regions of another
process. Multi-GPU cases run when two devices are visible."""

from __future__ import annotations

import multiprocessing as mp
import threading
import time

import pytest
import torch

from pplx_garden import _native
from pplx_garden.fabric_lib import MemoryRegionDescriptor, PageIndices, TransferEngine
from tests.test_fabric_cpu import Waiter

pytestmark = pytest.mark.gpu


@pytest.fixture()
def engines():
    a = TransferEngine(1, [0])
    b = TransferEngine(2, [0]) if False else TransferEngine(1, [0])
    yield a, b
    a.stop()
    b.stop()


def test_device_to_device_single_write(engines) -> None:
    a, b = engines
    dev = torch.device("cuda", 0)
    src = torch.randint(0, 255, (8 << 20,), dtype=torch.uint8, device=dev)
    dst = torch.zeros(8 << 20, dtype=torch.uint8, device=dev)
    hs, _ = a.register_tensor(src)
    _, dd = b.register_tensor(dst)
    torch.cuda.synchronize()
    for offset, length, dst_offset in ((0, 8 << 20, 0), (4096, 1 << 20, 65536), (16, 100_000, 48), (3, 1001, 5)):
        dst.zero_()
        torch.cuda.synchronize()
        w = Waiter()
        a.submit_write(hs, offset, length, None, dd, dst_offset, w.done, w.error)
        w.wait()
        torch.cuda.synchronize()
        assert torch.equal(dst[dst_offset:dst_offset + length], src[offset:offset + length])
        assert int(dst.count_nonzero()) <= length


def test_paged_kv_write_with_layer_notification(engines) -> None:
    """KV-cache shaped pages: 64 tokens x 8 heads x 128 dims, bf16, scattered source and
    destination page tables, one counted immediate per page."""
    a, b = engines
    dev = torch.device("cuda", 0)
    page_bytes = 64 * 8 * 128 * 2
    n_src, n_dst, n = 96, 128, 80
    src = torch.randn((n_src, page_bytes // 2), device=dev).to(torch.bfloat16)
    dst = torch.zeros((n_dst, page_bytes // 2), dtype=torch.bfloat16, device=dev)
    hs, _ = a.register_tensor(src)
    _, dd = b.register_tensor(dst)
    gen = torch.Generator().manual_seed(0)
    src_pages = torch.randperm(n_src, generator=gen)[:n].tolist()
    dst_pages = torch.randperm(n_dst, generator=gen)[:n].tolist()
    reached = threading.Event()
    b.set_imm_count_expected(0x100, n, reached.set)
    torch.cuda.synchronize()
    w = Waiter()
    a.submit_paged_writes(page_bytes, hs, PageIndices(src_pages), page_bytes, 0, dd, PageIndices(dst_pages),
                          page_bytes, 0, 0x100, w.done, w.error)
    w.wait()
    assert reached.wait(5)
    torch.cuda.synchronize()
    assert torch.equal(dst[dst_pages], src[src_pages])
    untouched = sorted(set(range(n_dst)) - set(dst_pages))
    assert int(dst[untouched].count_nonzero()) == 0


def test_host_device_writes(engines) -> None:
    a, b = engines
    dev = torch.device("cuda", 0)
    host_src = torch.randint(0, 255, (1 << 20,), dtype=torch.uint8).pin_memory()
    dev_dst = torch.zeros(1 << 20, dtype=torch.uint8, device=dev)
    host_dst = torch.zeros(1 << 20, dtype=torch.uint8).pin_memory()
    hs, _ = a.register_tensor(host_src)
    _, ddev = b.register_tensor(dev_dst)
    _, dhost = b.register_tensor(host_dst)
    hdev, _ = a.register_tensor(dev_dst)
    w = Waiter()
    a.submit_write(hs, 0, 1 << 20, None, ddev, 0, w.done, w.error)          # host -> device
    w.wait()
    torch.cuda.synchronize()
    assert torch.equal(dev_dst.cpu(), host_src)
    w = Waiter()
    a.submit_write(hdev, 128, 4096, None, dhost, 256, w.done, w.error)      # device -> host
    w.wait()
    assert torch.equal(host_dst[256:256 + 4096], host_src[128:128 + 4096])


def test_scalar_watcher_incremented_by_a_kernel(engines) -> None:
    a, _ = engines
    seen: list[tuple[int, int]] = []
    got = threading.Event()

    def on_change(old: int, new: int) -> bool:
        seen.append((old, new))
        got.set()
        return True

    watcher = a.alloc_scalar_watcher(on_change)
    cell = _native._tensor_from_ptr(watcher.ptr, 8, 0).view(torch.int64)
    cell.add_(41)                                     # a CUDA kernel writes the host-mapped word
    torch.cuda.synchronize()
    assert got.wait(5) and seen[0] == (0, 41)


def _gpu_server(conn, device_index: int) -> None:
    torch.cuda.set_device(device_index)
    engine = TransferEngine(1, [device_index])
    buf = torch.zeros(4 << 20, dtype=torch.uint8, device=torch.device("cuda", device_index))
    _, desc = engine.register_tensor(buf)
    torch.cuda.synchronize()
    reached = threading.Event()
    engine.set_imm_count_expected(0x33, 1, reached.set)
    conn.send(desc.as_bytes())
    ok = reached.wait(30)
    torch.cuda.synchronize()
    conn.send((ok, buf[:64].cpu().tolist(), int(buf.to(torch.int64).sum().item())))
    engine.stop()


@pytest.mark.parametrize("server_device", [0, 1])
def test_write_into_another_process(server_device: int) -> None:
    """The destination region lives in another process and is mapped through its CUDA IPC
    handle; with server_device 1 the bytes cross NVLink."""
    if torch.cuda.device_count() <= server_device:
        pytest.skip("needs a second GPU")
    ctx = mp.get_context("spawn")
    parent, child = ctx.Pipe()
    proc = ctx.Process(target=_gpu_server, args=(child, server_device))
    proc.start()
    try:
        desc = MemoryRegionDescriptor.from_bytes(parent.recv())
        engine = TransferEngine(1, [0])
        src = (torch.arange(4 << 20, device="cuda:0") % 253).to(torch.uint8)
        handle, _ = engine.register_tensor(src)
        torch.cuda.synchronize()
        w = Waiter()
        engine.submit_write(handle, 0, 4 << 20, 0x33, desc, 0, w.done, w.error)
        w.wait(30)
        ok, head, total = parent.recv()
        assert ok and head == src[:64].cpu().tolist() and total == int(src.to(torch.int64).sum().item())
        engine.stop()
    finally:
        proc.join(30)
        if proc.is_alive():
            proc.terminate()
