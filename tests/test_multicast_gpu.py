"""CUDA multicast objects (NVLS) across two processes and two GPUs: create, export / import,
add_device, bind_mem, map, one multimem.red on a flag word that both GPUs then find in their own
memory, and an orderly teardown (reference rust/cuda-lib/src/cumem.rs:525-610 exposes the same
objects and uses them nowhere).

Every rank unbinds and unmaps before it leaves, whatever happened in between: a process that
exits while its memory is still bound to a multicast object can fault the other GPUs."""

from __future__ import annotations

import pytest
import torch

from pplx_garden.distributed import ParallelLaunch

pytestmark = pytest.mark.gpu


def _worker(device, dp_group, global_group):
    from pplx_garden import _native
    from pplx_garden.native.cumem import CUMemAllocHandle, CUMemHandleKind, CUMulticastHandle

    rank, world = global_group.rank, global_group.size
    supported = all(global_group.all_gather_object(bool(CUMulticastHandle.supported(device))))
    if not supported:
        return "unsupported"
    kind = CUMemHandleKind.FileDescriptor
    mc = export = None
    try:
        if rank == 0:
            mc = CUMulticastHandle(world, 2 << 20, kind)
            export = mc.export()
    except Exception as exc:          # e.g. no fabric manager: nothing is bound yet, leaving is safe
        export = f"create failed: {exc}"
    export = global_group.all_gather_object(export)[0]
    if isinstance(export, str):
        return "unsupported"
    if rank != 0:
        mc = export.bind(device)
    mc.add_device(device)
    global_group.barrier()            # every device is in before anybody binds memory
    mem = CUMemAllocHandle(mc.size, device, kind)
    local = mem.map(device)
    words = local.to_tensor((mc.size // 4,), torch.int32)
    words.zero_()
    torch.cuda.synchronize(device)
    error = None
    seen = None
    mapping = None
    bound = False
    try:
        mc.bind_mem(mem)
        bound = True
        global_group.barrier()        # every rank's memory is bound before the first reduction
        mapping = mc.map(device)
        stream = torch.cuda.current_stream().cuda_stream
        _native.multimem_red_add_u32(mapping.data_ptr() + 4 * 7, rank + 1, stream)
        torch.cuda.synchronize(device)
        global_group.barrier()        # both reductions have been issued and have completed
        torch.cuda.synchronize(device)
        seen = int(words[7].item())
    except Exception as exc:          # reported after the teardown, never instead of it
        error = repr(exc)
    finally:
        torch.cuda.synchronize(device)
        global_group.barrier()        # nobody is still sending through the object
        if mapping is not None:
            mapping.unmap()
        if bound:
            mc.unbind()
        global_group.barrier()        # everybody is unbound before any memory goes away
        local.unmap()
    if error is not None:
        return error
    return seen


def test_multicast_object_round_trip_on_two_gpus() -> None:
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    results = ParallelLaunch(world_size=2).run(_worker)
    if all(r == "unsupported" for r in results):
        pytest.skip("multicast objects are not available on this machine")
    assert results == [3, 3], results      # 1 from rank 0 + 2 from rank 1, on both GPUs
