"""The allocation-free paged copy (csrc/noalloc/paged_copy_noalloc.h), called through its
exported C symbol, must move exactly the bytes that the transfer engine's regular paged write
moves. The regular path stages its page tables in a cudaMalloc'd buffer; this one is for
callers that are not allowed to allocate (a process whose memory is fully committed to a
KV-cache arena, a plugin without an allocator, a decode loop that cannot take the device-wide
synchronisation of cudaMalloc). Runs last so that a failure here cannot hide other tests."""

from __future__ import annotations

import ctypes
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu


def _load():
    lib_path = Path(__file__).resolve().parent.parent / "pplx_garden" / "libpplx_noalloc.so"
    assert lib_path.exists(), "libpplx_noalloc.so is not built: run python build.py"
    lib = ctypes.CDLL(str(lib_path))
    lib.pplx_paged_copy_noalloc.restype = ctypes.c_int
    lib.pplx_paged_copy_noalloc.argtypes = [
        ctypes.c_void_p, ctypes.c_void_p, ctypes.POINTER(ctypes.c_uint32), ctypes.POINTER(ctypes.c_uint32),
        ctypes.c_uint32, ctypes.c_uint64, ctypes.c_uint64, ctypes.c_uint64, ctypes.c_uint64, ctypes.c_uint64,
        ctypes.c_void_p,
    ]
    lib.pplx_paged_copy_noalloc_max_pages.restype = ctypes.c_uint32
    lib.pplx_noalloc_last_error.restype = ctypes.c_char_p
    return lib


def _reference_copy(src, dst, src_pages, dst_pages, length, src_stride, dst_stride, src_off, dst_off):
    """The existing entry point: a paged write through the transfer engine."""
    import threading

    from pplx_garden.fabric_lib import PageIndices, TransferEngine

    a, b = TransferEngine(1, [0]), TransferEngine(1, [0])
    try:
        hs, _ = a.register_tensor(src)
        _, dd = b.register_tensor(dst)
        done, errors = threading.Event(), []
        a.submit_paged_writes(length, hs, PageIndices(src_pages), src_stride, src_off, dd,
                              PageIndices(dst_pages), dst_stride, dst_off, None, done.set,
                              lambda e: (errors.append(e), done.set()))
        assert done.wait(20) and not errors, errors
        torch.cuda.synchronize()
    finally:
        a.stop()
        b.stop()


def test_no_alloc_paged_copy_matches_the_engine_twice_in_a_row() -> None:
    lib = _load()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    page = 64 * 8 * 128 * 2                     # one KV page: 64 tokens x 8 heads x 128 dims, bf16
    n_src, n_dst = 48, 64
    src = torch.randint(0, 255, (n_src * page,), dtype=torch.uint8, device=dev)
    gen = torch.Generator().manual_seed(7)
    stream = torch.cuda.current_stream().cuda_stream
    calls = [
        dict(n=40, length=page, src_off=0, dst_off=0),             # aligned: 16-byte vectors
        dict(n=17, length=page // 2 - 3, src_off=5, dst_off=9),    # odd sizes: byte path, fewer pages
    ]
    for call in calls:                          # two calls in a row share the static page tables
        n = call["n"]
        src_pages = torch.randperm(n_src, generator=gen)[:n].tolist()
        dst_pages = torch.randperm(n_dst, generator=gen)[:n].tolist()
        want = torch.zeros(n_dst * page, dtype=torch.uint8, device=dev)
        got = torch.zeros(n_dst * page, dtype=torch.uint8, device=dev)
        torch.cuda.synchronize()
        _reference_copy(src, want, src_pages, dst_pages, call["length"], page, page,
                        call["src_off"], call["dst_off"])
        sp = (ctypes.c_uint32 * n)(*src_pages)
        dp = (ctypes.c_uint32 * n)(*dst_pages)
        rc = lib.pplx_paged_copy_noalloc(src.data_ptr(), got.data_ptr(), sp, dp, n, page, page,
                                         call["src_off"], call["dst_off"], call["length"], stream)
        assert rc == 0, lib.pplx_noalloc_last_error().decode()
        torch.cuda.synchronize()
        assert torch.equal(got, want)
        assert int(got.count_nonzero()) > 0


def test_no_alloc_paged_copy_rejects_oversized_requests() -> None:
    lib = _load()
    torch.cuda.set_device(0)
    limit = lib.pplx_paged_copy_noalloc_max_pages()
    assert limit == 65536
    buf = torch.zeros(4096, dtype=torch.uint8, device="cuda:0")
    pages = (ctypes.c_uint32 * 1)(0)
    rc = lib.pplx_paged_copy_noalloc(buf.data_ptr(), buf.data_ptr(), pages, pages, limit + 1, 0, 0, 0, 0, 16, None)
    assert rc == -1 and b"exceed the limit" in lib.pplx_noalloc_last_error()


def test_no_alloc_paged_copy_with_pinned_page_tables() -> None:
    """Page tables in pinned host memory are read when the stream gets to them, not when the
    call returns: the caller keeps them unchanged until a synchronisation, as the header says."""
    lib = _load()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    page, n = 4096, 24
    src = torch.randint(0, 255, (n * page,), dtype=torch.uint8, device=dev)
    got = torch.zeros(n * page, dtype=torch.uint8, device=dev)
    order = torch.randperm(n, generator=torch.Generator().manual_seed(3)).to(torch.int32)
    src_tab = torch.arange(n, dtype=torch.int32).pin_memory()
    dst_tab = order.clone().pin_memory()
    u32p = ctypes.POINTER(ctypes.c_uint32)
    rc = lib.pplx_paged_copy_noalloc(src.data_ptr(), got.data_ptr(),
                                     ctypes.cast(src_tab.data_ptr(), u32p),
                                     ctypes.cast(dst_tab.data_ptr(), u32p), n, page, page, 0, 0, page,
                                     torch.cuda.current_stream().cuda_stream)
    assert rc == 0, lib.pplx_noalloc_last_error().decode()
    torch.cuda.synchronize()        # only now may src_tab / dst_tab change
    want = torch.zeros_like(got)
    want.view(n, page)[order.long().to(dev)] = src.view(n, page)
    assert torch.equal(got, want)
