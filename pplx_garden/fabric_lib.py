"""The transfer engine: registered memory regions, one-sided single / paged / scatter
writes with immediate-value notification, two-sided messages and scalar watchers.

Same names as the reference's python/pplx_garden/fabric_lib.py:3-12. On a machine without
RDMA NICs the engine's domains are the intra-box provider: GPU-to-GPU writes run as a
peer-copy kernel over NVLink, host memory and control messages go through unix sockets.
"""

from pplx_garden._native import (
    DomainAddress as DomainAddress,
    DomainInfo as DomainInfo,
    ImmCounter as ImmCounter,
    MemoryRegionDescriptor as MemoryRegionDescriptor,
    MemoryRegionHandle as MemoryRegionHandle,
    PageIndices as PageIndices,
    ScatterTarget as ScatterTarget,
    TopologyGroup as TopologyGroup,
    TransferCounter as TransferCounter,
    TransferEngine as TransferEngine,
    TransferEngineBuilder as TransferEngineBuilder,
    UvmWatcher as UvmWatcher,
)
